// The transport under the active-message context: what libucp is to the
// reference (ucp_worker_progress, ucp_am_send_nbx, ucp_am_recv_data_nbx,
// listeners and endpoints; ucx_context/ucx_connection.cpp:184-242, 353-450).
//
// Control plane: non-blocking TCP sockets polled by the single worker thread.
// Every active message is a frame {fixed 40-byte frame header, AM header bytes,
// segment sizes, payload}. Small host payloads travel inline (eager). Larger
// ones, scatter-gather ones and every device payload use a rendezvous:
//
//   host memory:    RTS -> (receiver posts its buffer) -> CTS -> DATA, read by
//                   the receiver straight into the posted buffer;
//   device memory:  RTS carries one PeerRegionDesc (CUDA IPC export) per
//                   segment; the receiver maps the regions and launches the
//                   transfer kernel that reads the sender's memory over NVLink
//                   into the posted device buffer, then answers FIN. The kernel
//                   signals completion by writing a flag in mapped pinned host
//                   memory that progress() polls. When the regions cannot be
//                   mapped (or the receiver wants host memory) the payload is
//                   staged through host memory with the host protocol.
//
// The Worker is single-threaded: every method is called from the thread that
// runs progress().
#pragma once

#include <netinet/in.h>
#include <sys/socket.h>

#include <chrono>
#include <cstdint>
#include <deque>
#include <functional>
#include <list>
#include <sys/uio.h>

#include <atomic>
#include <memory>
#include <mutex>
#include <set>
#include <string>
#include <unordered_map>
#include <vector>

#include "eux/ucxx/cuda/ucx_cuda_memory_manager.hpp"
#include "kernels/eux_kernels.h"
#include "eux/ucxx/ucx_context_def.h"
#include "eux/ucxx/shm_channel.hpp"
#include "eux/ucxx/ucx_memory_resource.hpp"
#include "eux/ucxx/ucx_send_attr.hpp"
#include "eux/ucxx/ucx_status.hpp"

namespace eux::ucxx::transport {

class Worker;
class Endpoint;

using Completion = std::function<void(int status)>;

// Test shim for fault injection on the host: when set, every outgoing frame is shown to the hook
// (the sending worker's name, the frame type, the message id); a frame for which it returns true
// is dropped as if the wire had lost it (its local completion still fires). Process-wide; tests
// install it, run a scenario, and clear it again with an empty function.
using FaultHook = std::function<bool(const std::string& worker_name, uint8_t frame_type, uint64_t msg_id)>;
void set_fault_hook(FaultHook hook);

// A device payload that arrived eagerly lies in a slot of the receive ring and is handed to the application as
// it lies; the slot goes back to the sender when the application drops the buffer. The contract of the C++
// interface is that dropping it means being done with it, work queued on the GPU included (a handler that
// launches a kernel on the payload keeps the payload until the kernel has finished, as the handlers that return
// schedule_when_flag senders do). A layer whose users cannot keep that contract (the Python binding: a tensor
// is dropped when its last reference goes, whatever is still queued on the tensor library's stream) installs a
// hook that is asked at every drop: it returns kConsumerDone (hand the slot back now: nothing is queued), or
// records an event behind the queued work, stores it in *event (a cudaEvent_t that the transport destroys) and
// returns kConsumerEvent: the slot goes back when the event has completed.
enum ConsumerState : int { kConsumerDone = 0, kConsumerEvent = 1 };
using ConsumerEventHook = int (*)(int device, void** event);
void set_consumer_event_hook(ConsumerEventHook hook);

// True when a worker with this uid (the random number in its address) is alive in this process. A peer
// is taken to be "this process" only on that evidence, never on a pid that came over the wire.
bool is_live_local_uid(uint64_t uid);

constexpr uint32_t kFrameMagic = 0x46585545u;  // "EUXF"
// Most bytes an active-message header may have (a serialized RPC header with its parameters). A longer one is
// refused by the sender before it leaves and by the receiver when it is announced.
inline constexpr size_t kMaxHeaderLen = size_t(16) << 20;
enum FrameType : uint8_t {
  kHello = 1,
  kHelloAck = 2,
  kAmEager = 3,
  kAmRts = 4,
  kRndvCts = 5,
  kRndvData = 6,
  kRndvFin = 7,
  kClose = 8,
  kDevRing = 9,     // same-host peers with GPUs: "this is my device receive ring" (one PeerRegionDesc + geometry)
  kAmDevEager = 10, // active message whose small device payload is being pushed into the receiver's ring slot
};
enum FrameFlags : uint8_t {
  kFlagDeviceRegions = 1,  // RTS carries PeerRegionDesc per segment
  kFlagStage = 2,          // CTS: send the payload through host memory
  kFlagShmOffer = 4,       // HELLO: the name of a shared-memory channel follows the address
  kFlagShmAccept = 8,      // HELLO_ACK: the channel is mapped; frames travel through it from now on
  kFlagPushOk = 16,        // RTS: the sender can push the payload itself and signal through the shared flag page
  kFlagFromSender = 64,    // FIN: sent by the sender of the message (send withdrawn / cannot push), not by its receiver
  kFlagLayout = 128,       // RTS: the payload is a strided view; one region (its span) and a WireLayout follow
  kFlagPush = 32,          // CTS: "push it here": the receiver's regions follow, status = flag word, payload_len = flag value
};

#pragma pack(push, 1)
struct FrameHeader {
  uint32_t magic = kFrameMagic;
  uint8_t type = 0;
  uint8_t flags = 0;
  uint16_t am_id = 0;
  uint32_t header_len = 0;  // AM header bytes that follow
  uint32_t seg_count = 0;   // number of payload segments described after the AM header
  uint64_t payload_len = 0; // total payload bytes (inline for eager / DATA)
  uint64_t msg_id = 0;
  uint32_t mem_type = 0;    // ucx_memory_type of the sender's payload
  int32_t status = 0;       // FIN
};
#pragma pack(pop)
static_assert(sizeof(FrameHeader) == 40);

// How the elements of a strided payload lie in the sender's region (see ucx_send_attr.hpp); follows the
// region descriptor of an RTS with kFlagLayout.
struct WireLayout {
  int32_t ndim = 0;
  uint16_t elem_size = 0;                  // of an element in the sender's memory
  uint8_t src_dtype = 0, dst_dtype = 0;    // see UcxSendAttr
  int64_t shape[kSendAttrMaxDims] = {0};
  int64_t stride[kSendAttrMaxDims] = {0};
  uint64_t span_bytes = 0;
};
static_assert(sizeof(WireLayout) == 144);
using SendHint = UcxSendAttr;

// Address of a worker, exchanged out of band (what get_ucp_address() returns).
struct WorkerAddress {
  uint32_t magic = 0x41585545u;  // "EUXA"
  uint32_t ipv4 = 0;             // network byte order
  uint16_t port = 0;             // host byte order
  uint16_t reserved = 0;
  uint32_t pid = 0;
  int32_t device = -1;
  uint64_t uid = 0;
  char name[32] = {0};
  std::vector<std::byte> serialize() const;
  static bool parse(const std::byte* p, size_t n, WorkerAddress* out);
};

// An incoming active message as seen by the context (UcxAmDesc in the reference).
struct AmArrival {
  Endpoint* ep = nullptr;
  void* header = nullptr;   // HOST memory from the worker's memory resource; ownership passes to the callee
  size_t header_len = 0;
  void* data = nullptr;     // eager payload, HOST memory from the memory resource; ownership passes to the callee
  size_t data_len = 0;      // total payload bytes
  bool rndv = false;
  uint64_t msg_id = 0;
  uint32_t seg_count = 0;   // > 0 only for scatter-gather sends
  ucx_memory_type_t sender_mem_type = ucx_memory_type::HOST;
  // Where `data` lives. HOST: memory of the worker's resource, to be deallocated by the callee.
  // CUDA: a slot of this worker's device receive ring; the callee drops `data_keep` when it is done
  // with the bytes (that returns the slot to the sender), and never deallocates `data`.
  ucx_memory_type_t data_mem_type = ucx_memory_type::HOST;
  std::shared_ptr<void> data_keep;
};

struct ConnRequest {
  int fd = -1;
  uint64_t client_id = 0;
  std::string peer_name;   // "ip:port" of the remote socket
  std::string worker_name; // name of the remote worker
  WorkerAddress remote{};
  std::chrono::steady_clock::time_point arrival;
  std::vector<char> pending;  // bytes already read past the HELLO frame
  std::string shm_name;       // shared-memory channel offered by the peer, if any
};

struct WorkerOptions {
  std::string name = "default";
  uint64_t client_id = 0;
  int device = -1;               // CUDA device of this worker, -1 = none
  size_t eager_limit = 8192;     // payloads below this travel inline (host memory)
  size_t send_copy_limit = 8192; // inline payloads up to this size are copied, so the send completes at once
  bool use_shm = true;           // peers on this host talk through shared-memory rings (EUX_SHM=0 turns it off)
  // Device payloads up to this size go out eagerly: the sender's kernel (one CTA of a batched launch up to
  // 64 KiB, a launch of its own above) stores them into the peer's device receive ring (32 slots of a quarter
  // of this limit, at most 1 MiB each; a payload takes a run of consecutive slots, up to 16) and raises a flag
  // the peer's host thread polls. No RTS, no FIN, and the receiver asks no memory policy: the payload is handed
  // on where it lies. 0 turns the path off (EUX_DEV_EAGER_LIMIT); at most 16 MiB.
  size_t dev_eager_limit = size_t(16) << 20;
  // Device payloads from this size on are pushed by the sender's kernel (the receiver answers the RTS with
  // its own regions) instead of pulled by the receiver's: with traffic in both directions stores keep
  // the links fuller than loads. 0 turns pushing off (EUX_PUSH_THRESH).
  size_t push_threshold = size_t(4) << 20;
};

class Endpoint {
 public:
  enum class State { kConnecting, kHelloSent, kConnected, kClosed, kFailed };
  uint64_t id() const { return reinterpret_cast<uint64_t>(this); }
  State state() const { return state_; }
  const std::string& peer_name() const { return peer_name_; }
  const std::string& remote_worker_name() const { return remote_.name_str; }
  uint32_t remote_pid() const { return remote_.addr.pid; }
  int remote_device() const { return remote_.addr.device; }
  uint64_t remote_client_id() const { return remote_client_id_; }
  void* user_data = nullptr;  // the UcxConnection that wraps this endpoint

 private:
  friend class Worker;
  struct SendItem {
    std::vector<char> owned;      // frame header + AM header + metadata (+ copied payload)
    std::vector<ucx_buffer_t> segs;  // user memory that follows `owned` on the wire
    size_t seg_idx = 0, seg_off = 0, owned_off = 0;
    Completion done;              // fired when the last byte is written (may be empty)
    std::shared_ptr<void> keep;   // staging buffer kept alive until written
    bool switch_to_shm = false;   // the HELLO_ACK that accepts a channel: what follows it goes through the rings
  };
  struct PendingSend {             // rendezvous send waiting for CTS / FIN
    std::vector<ucx_buffer_t> segs;
    ucx_memory_type_t mem_type;
    Completion done;
    std::shared_ptr<const SendHint> layout;  // set when segs[0] is a strided view (its size is the dense size)
    std::shared_ptr<void> keep;              // a packed copy that stands in for the user's memory
  };
  struct PendingRecv {             // posted rendezvous receive waiting for DATA
    std::vector<ucx_buffer_t> segs;
    ucx_memory_type_t mem_type;
    Completion done;
    std::shared_ptr<void> bounce;  // host staging when the destination is device memory
    std::vector<ucx_buffer_t> dev_dsts;  // the real destinations behind the bounce buffer
    size_t total = 0;
  };
  struct RtsInfo {                 // what an RTS said, kept until the receive is posted
    uint64_t payload_len = 0;
    ucx_memory_type_t mem_type = ucx_memory_type::HOST;
    std::vector<uint64_t> seg_sizes;
    std::vector<PeerRegionDesc> regions;
    bool push_ok = false;          // the sender offered to push the payload itself
    bool has_layout = false;       // the one region holds a strided view: gather it as `layout` says
    WireLayout layout;
  };
  struct RemoteInfo {
    WorkerAddress addr{};
    std::string name_str;
  };

  Worker* worker_ = nullptr;
  int fd_ = -1;
  // Same-host peers whose workers manage device memory: a Unix socket beside the control channel, over
  // which file descriptors of cuMemCreate allocations are passed (a descriptor cannot travel in a frame).
  int fd_chan_ = -1;
  std::set<uint64_t> vmm_sent_;  // allocations (by this process's number) whose descriptor the peer already has
  State state_ = State::kConnecting;
  std::string peer_name_;
  RemoteInfo remote_;
  uint64_t remote_client_id_ = 0;
  uint64_t next_msg_id_ = 1;
  std::deque<SendItem> sendq_;
  bool want_write_ = false;
  // receive state machine
  std::vector<char> rbuf_;         // bytes read but not yet consumed
  size_t rpos_ = 0;
  bool direct_active_ = false;     // DATA body is being read straight into a posted receive
  uint64_t direct_msg_ = 0;
  size_t direct_seg_ = 0, direct_off_ = 0, direct_left_ = 0, direct_total_ = 0;
  std::unordered_map<uint64_t, PendingSend> pending_sends_;
  std::unordered_map<uint64_t, PendingRecv> pending_recvs_;
  std::unordered_map<uint64_t, RtsInfo> rts_;
  Completion on_connected_;
  bool auto_accepted_ = false;
  std::shared_ptr<ShmChannel> shm_;  // offered or mapped channel (buffers handed to the application may outlive the endpoint)
  bool shm_active_ = false;          // frames go through shm_ instead of the socket
  // ---- device channel: set up after the shared-memory channel when both workers drive a GPU ----
  struct DevRing {                   // this side's receive ring in device memory
    UcxMemoryResourceManager* mr = nullptr;
    void* base = nullptr;
    size_t bytes = 0;
    uint32_t slot_bytes = 0;
    ~DevRing();
  };
  bool dev_tried_ = false;           // set-up was attempted (whatever came of it)
  bool flags_registered_ = false;    // the channel's flag pages are registered with CUDA in this process
  uint64_t* out_flags_dev_ = nullptr;  // device alias of shm_->out_flags()
  std::shared_ptr<DevRing> rx_ring_;   // slots the peer pushes eager payloads into
  char* tx_ring_ = nullptr;            // the peer's ring, mapped here
  uint32_t tx_slots_ = 0, tx_slot_bytes_ = 0;
  uint64_t tx_free_ = 0;               // bit i: slot i of the peer's ring is free
  uint64_t tx_seq_ = 0;                // flag values of eager pushes (per endpoint, increasing)
  uint64_t push_seq_ = 0;              // flag values handed out for payloads the peer pushes to this side
  uint32_t push_inflight_ = 0;
  bool await_dev_ring_ = false;        // connect completion held back until the peer's kDevRing frame
  std::chrono::steady_clock::time_point dev_ring_deadline_{};
  bool staged_logged_ = false;       // the "staged through the host" line was printed for this endpoint
};

class Worker {
 public:
  // 0 keeps the current value
  void set_limits(size_t eager_limit, size_t send_copy_limit) {
    if (eager_limit) opt_.eager_limit = eager_limit;
    if (send_copy_limit) opt_.send_copy_limit = send_copy_limit;
  }
  Worker(UcxMemoryResourceManager& mr, const WorkerOptions& opt);
  ~Worker();
  Worker(const Worker&) = delete;

  // ---- callbacks into the context (set once, before progress()) ----
  std::function<void(AmArrival&&)> on_am;                     // active message arrived
  std::function<void(ConnRequest&&)> on_conn_request;         // HELLO on an explicit listener
  std::function<void(Endpoint*)> on_auto_accept;              // connection made through the worker address
  std::function<void(Endpoint*, int status)> on_ep_error;     // endpoint failed / closed by peer

  // Poll sockets and device completions once; returns the number of events handled.
  int progress();
  // steady_clock as read at the start of the last progress() call
  std::chrono::steady_clock::time_point last_progress_time() const noexcept { return last_progress_; }

  WorkerAddress address() const { return addr_; }
  const WorkerOptions& options() const { return opt_; }
  UcxMemoryResourceManager& mr() { return mr_; }

  // Explicit listener (accept_endpoint); returns a UCS status.
  int listen(const sockaddr* addr, socklen_t len);
  int listen(uint16_t port);
  void stop_listening();

  // Start connecting; `done(status)` fires from progress() when the handshake ends.
  Endpoint* connect(const sockaddr* dst, socklen_t len, const sockaddr* src, socklen_t src_len, Completion done, int* status);
  Endpoint* connect(const WorkerAddress& addr, Completion done, int* status);
  Endpoint* accept(ConnRequest&& req, int* status);
  void reject(ConnRequest&& req);
  void close(Endpoint* ep, bool notify_peer = true);
  void destroy(Endpoint* ep);  // free a closed/failed endpoint

  // Active message send. `segs` must stay valid until `done` fires. Returns UCS_OK when
  // the send completed inline (done is NOT called), UCS_INPROGRESS when it will complete
  // later, or an error (done is NOT called).
  // `hint` (device payloads only; see ucx_send_attr.hpp) may describe segs[0] as a strided view and name an
  // event after which the payload is complete.
  int am_send(Endpoint* ep, const void* header, size_t header_len, const ucx_buffer_t* segs, size_t seg_count,
              ucx_memory_type_t mem_type, bool force_rndv, Completion done, uint64_t* msg_id_out = nullptr,
              std::shared_ptr<const SendHint> hint = nullptr);
  // Complete a rendezvous receive into `segs` (of `mem_type`). Same return convention.
  // `ready` (device destinations): an event after which the posted buffers may be written. Memory fresh from a
  // stream-ordered allocator may still be in use by work queued before it was handed out; the transport's own
  // kernel waits for the event on the device, and a peer is asked to push only once it has completed.
  int rndv_recv(Endpoint* ep, uint64_t msg_id, const ucx_buffer_t* segs, size_t seg_count, ucx_memory_type_t mem_type,
                Completion done, std::shared_ptr<const SendHint> ready = nullptr);
  // Drop a rendezvous message that will never be received (tells the sender).
  void rndv_discard(Endpoint* ep, uint64_t msg_id);
  // Segment sizes announced by the sender of a rendezvous message (empty if unknown).
  std::vector<uint64_t> rndv_segment_sizes(Endpoint* ep, uint64_t msg_id) const;
  // Withdraw a pending operation. true: it is gone and its callback will never fire;
  // false: it is past the point of no return and will complete by itself.
  bool cancel_send(Endpoint* ep, uint64_t msg_id);
  bool cancel_recv(Endpoint* ep, uint64_t msg_id);

  size_t endpoint_count() const { return eps_.size(); }

  // Counters of the decisions that cost performance or that refuse input; read from the worker's thread.
  struct Stats {
    uint64_t frames_refused = 0;   // frames whose sizes were beyond the limits (the endpoint was failed)
    uint64_t regions_ignored = 0;  // device regions announced by a peer that did not prove it is on this host
    uint64_t device_pulls = 0;     // device payloads moved by the transfer kernel
    uint64_t device_staged = 0;    // device payloads that went through host memory instead
    uint64_t truncated = 0;        // DATA frames whose length was not the posted one
    uint64_t device_eager_sent = 0;  // small device payloads pushed into a peer's ring
    uint64_t device_eager_recv = 0;  // ... and received through this worker's rings
    uint64_t device_pushes = 0;      // large device payloads pushed by this worker's kernel on a CTS(push)
    uint64_t device_push_recv = 0;   // ... and received that way
    uint64_t kernel_launches = 0;    // launches of the transfer kernels by this worker
    uint64_t device_gathers = 0;     // strided payloads gathered by the transfer itself (into a ring slot, or by a pull)
    uint64_t device_packs = 0;       // ... and those packed into a dense copy first because they could not be
    uint64_t sends_held = 0;         // announcements held back until the payload's producer had finished
    uint64_t vmm_fds_sent = 0;       // cuMemCreate allocations handed to a peer as file descriptors
    uint64_t vmm_fds_recv = 0;       // ... and mapped from descriptors that a peer handed over
  };
  const Stats& stats() const { return stats_; }

 private:
  struct Listener {
    int fd = -1;
    bool implicit = false;
  };
  struct HelloWait {  // accepted socket that has not sent its HELLO yet
    int fd;
    bool implicit;
    std::string peer;
    std::vector<char> buf;
    std::chrono::steady_clock::time_point since;
  };
  struct DeviceOp {   // transfer kernel in flight
    uint64_t seq;
    Endpoint* ep;
    uint64_t msg_id;
    Completion done;
    bool send_fin = true;  // a pull answers the sender with FIN; a push or an eager send tells nobody
    std::shared_ptr<const void> keep = nullptr;  // what the kernel reads from or waits on, if it is the transport's to keep
  };
  struct HeldSend {   // a frame that announces device memory whose producer has not finished yet
    Endpoint* ep;
    std::shared_ptr<const SendHint> hint;
    Endpoint::SendItem item;
    uint64_t msg_id = 0;  // of an RTS (0: a CTS, whose wait has a deadline of its own)
    std::chrono::steady_clock::time_point deadline{};
  };
  struct EagerWait {  // kAmDevEager frame received, its payload still on the way into the ring slot
    Endpoint* ep;
    std::shared_ptr<ShmChannel> shm;
    std::shared_ptr<Endpoint::DevRing> ring;
    uint32_t slot;
    uint64_t seq;
    AmArrival arrival;
    std::chrono::steady_clock::time_point deadline;
  };
  struct PushWait {   // CTS(push) sent: the peer's kernel writes into the posted buffers and then the flag word
    Endpoint* ep;
    std::shared_ptr<ShmChannel> shm;
    uint64_t msg_id;
    uint32_t word;
    uint64_t value;
    Completion done;
    Endpoint::RtsInfo info;               // kept for the fall-back when the peer cannot push after all
    std::vector<ucx_buffer_t> segs;
    std::chrono::steady_clock::time_point deadline;
    std::shared_ptr<const SendHint> ready;  // kept for the fall-back (and owns the event until then)
  };
  Endpoint* new_endpoint(int fd);
  void fail(Endpoint* ep, int status);
  void handle_readable(Endpoint* ep);
  void handle_writable(Endpoint* ep);
  bool parse_frames(Endpoint* ep);
  void dispatch_frame(Endpoint* ep, const FrameHeader& fh, const char* body);
  void enqueue(Endpoint* ep, Endpoint::SendItem&& item);
  void flush(Endpoint* ep);
  void send_control(Endpoint* ep, uint8_t type, uint8_t flags, uint64_t msg_id, int32_t status = 0);
  void send_hello(Endpoint* ep, uint8_t type, uint8_t flags = 0, const std::string& shm_name = {});
  void accept_pending(Listener& l);
  void poll_hellos();
  void start_data_send(Endpoint* ep, uint64_t msg_id, bool staged);
  int device_pull(Endpoint* ep, uint64_t msg_id, Endpoint::RtsInfo& info, const ucx_buffer_t* segs, size_t seg_count,
                  Completion& done, const std::shared_ptr<const SendHint>& ready);
  bool peer_is_this_process(const Endpoint* ep) const;
  bool peer_is_local(const Endpoint* ep) const;
  bool ensure_device();
  void poll_device();
  void poll_held_sends();
  static void drain_slot_releases();
  std::deque<HeldSend> held_sends_;
  // strided source -> dense device buffer of this worker's pool (the fallback when the gather cannot be fused
  // into the transfer); null on failure. Returns after the copy has finished.
  std::shared_ptr<void> pack_local(const SendHint& h, const void* src);
  static void fill_gather(eux_xfer_desc* d, const WireLayout& l);
  void setup_device_channel(Endpoint* ep);
  // file-descriptor channel (see Endpoint::fd_chan_)
  void open_fd_listener();
  void accept_fd_channels();
  void connect_fd_channel(Endpoint* ep);
  void close_fd_channel(Endpoint* ep);
  bool send_vmm_fd(Endpoint* ep, const PeerRegionDesc& d);
  void drain_fd_channel(Endpoint* ep);
  // Describe up to `limit` bytes of the segments for this peer, one descriptor per allocation touched, and
  // make sure the peer holds what it needs to map them. False (and `out` empty): take the staged protocol.
  bool export_for_peer(Endpoint* ep, const ucx_buffer_t* segs, size_t seg_count, uint64_t limit, std::vector<PeerRegionDesc>* out);
  void* import_from_peer(Endpoint* ep, const PeerRegionDesc& d);
  int fd_listen_ = -1;
  std::string fd_path_;
  void finish_connect(Endpoint* ep);
  void teardown_device_channel(Endpoint* ep);
  void on_dev_ring(Endpoint* ep, const FrameHeader& fh, const char* body);
  void on_dev_eager(Endpoint* ep, const FrameHeader& fh, const char* body);
  void on_push_cts(Endpoint* ep, const FrameHeader& fh, const char* body);
  int dev_eager_send(Endpoint* ep, const void* header, size_t header_len, const ucx_buffer_t& seg, ucx_memory_type_t mem_type,
                     uint64_t msg_id, Completion& done, const std::shared_ptr<const SendHint>& hint);
  int request_push(Endpoint* ep, uint64_t msg_id, Endpoint::RtsInfo& info, const ucx_buffer_t* segs, size_t seg_count, Completion& done,
                   const std::shared_ptr<const SendHint>& ready);
  int launch_pieces(const std::vector<std::pair<const void*, void*>>& ptrs, const std::vector<size_t>& lens, uint64_t* flag, uint64_t flag_value,
                    uint64_t* flag2, uint64_t flag2_value);
  void flush_pull_batch();
  void update_interest(Endpoint* ep);

  UcxMemoryResourceManager& mr_;
  UcxCudaMemoryResourceManager* cuda_mr_ = nullptr;  // non-null when the manager can export/import
  WorkerOptions opt_;
  std::vector<Endpoint*> shm_eps_;  // endpoints whose rings are polled by progress()
  void activate_shm(Endpoint* ep);
  ssize_t io_read(Endpoint* ep, void* buf, size_t n);
  ssize_t io_readv(Endpoint* ep, const struct iovec* iov, int cnt);
  ssize_t io_writev(Endpoint* ep, const struct iovec* iov, int cnt);
  WorkerAddress addr_{};
  int epfd_ = -1;
  std::chrono::steady_clock::time_point last_epoll_{};
  std::chrono::steady_clock::time_point last_progress_{};
  std::vector<Listener> listeners_;
  std::list<HelloWait> hellos_;
  std::unordered_map<Endpoint*, std::unique_ptr<Endpoint>> eps_;
  std::vector<Endpoint*> graveyard_;
  std::vector<Endpoint*> reparse_;
  // device side
  bool device_ready_ = false, device_failed_ = false;
  void* stream_ = nullptr;
  uint64_t* flag_host_ = nullptr;  // mapped pinned memory written by kernels
  uint64_t* flag_dev_ = nullptr;
  uint32_t* counter_dev_ = nullptr;
  bool bulk_used_ = false;  // this worker has put pushes on the process-wide stream of its device
  uint64_t device_seq_ = 0;
  std::deque<DeviceOp> device_ops_;
  // Small single-segment pulls wait here until the end of the current pass of the loop and then leave in
  // one launch (one CTA each). Every transfer owns the flag slot `seq % kFlagSlots` until it is reaped.
  static constexpr size_t kFlagSlots = 512;
  static constexpr size_t kBatchMaxBytes = size_t(256) << 10;
  std::vector<eux_pull_item> pull_batch_;
  std::vector<Endpoint*> awaiting_ring_;
  std::deque<EagerWait> eager_waits_;
  std::deque<PushWait> push_waits_;
  Stats stats_;
  void note_staged(Endpoint* ep, const char* why);
};

}  // namespace eux::ucxx::transport
