// Avro codec, request serialisation, double-buffered file streams, AxonStorage (CPU only).
#include <unistd.h>

#include <cstring>

#include "check.hpp"
#include "eux/axon/storage/avro_schema.hpp"
#include "eux/axon/storage/avro_serialization.hpp"
#include "eux/axon/storage/axon_storage.hpp"
#include "eux/axon/storage/unifex_io.hpp"

using namespace eux::axon::storage;
using namespace eux::rpc;
using eux::axon::utils::AxonRequest;
using eux::ucxx::DefaultUcxMemoryResourceManager;
using eux::ucxx::UcxBuffer;
using eux::ucxx::UcxBufferVec;
namespace ex = eux::exec;

static std::string tmpdir() {
  char dir[] = "/tmp/eux_storage_XXXXXX";
  if (!mkdtemp(dir)) throw std::runtime_error("mkdtemp");
  return dir;
}

EUX_TEST(avro_primitives_golden) {
  std::vector<uint8_t> out;
  avro::Encoder e(out);
  e.put_long(0);
  e.put_long(-1);
  e.put_long(1);
  e.put_long(-64);
  e.put_long(64);
  e.put_string("foo");
  // zig-zag varints from the Avro specification: 0->00, -1->01, 1->02, -64->7f, 64->80 01; "foo" -> 06 66 6f 6f
  const uint8_t want[] = {0x00, 0x01, 0x02, 0x7f, 0x80, 0x01, 0x06, 'f', 'o', 'o'};
  CHECK_EQ(out.size(), sizeof(want));
  CHECK(std::memcmp(out.data(), want, sizeof(want)) == 0);
  avro::Decoder d(out.data(), out.size());
  CHECK_EQ(d.get_long(), 0);
  CHECK_EQ(d.get_long(), -1);
  CHECK_EQ(d.get_long(), 1);
  CHECK_EQ(d.get_long(), -64);
  CHECK_EQ(d.get_long(), 64);
  CHECK(d.get_string() == "foo");
  CHECK(d.at_end());
  CHECK_THROWS(d.get_long());
  CHECK(AvroSchema::GetArrivalRequestSchema().find("\"name\":\"AxonRequest\"") != std::string_view::npos);
}

static std::shared_ptr<AxonRequest> make_request(DefaultUcxMemoryResourceManager& mr, uint32_t id, int payload_kind) {
  RpcRequestHeader h;
  h.session_id = session_id_t{7};
  h.request_id = request_id_t{id};
  h.function_id = function_id_t{0xfffffff0u};  // exercises the sign handling of Avro's int
  h.hlc = HybridLogicalClock(1000 + id, uint16_t(id));
  h.workflow_id = workflow_id_t{3};
  h.AddParam(true);
  h.AddParam(int16_t(-7));
  h.AddParam(uint32_t(4000000000u));
  h.AddParam(uint64_t(1) << 63);
  h.AddParam(1.5f);
  h.AddParam(-2.5);
  h.AddParam(data::string("text"));
  h.AddParam(data::vector<bool>{true, false});
  h.AddParam(data::vector<uint8_t>{1, 2, 255});
  h.AddParam(data::vector<int64_t>{-1, 1ll << 40});
  h.AddParam(data::vector<float>{0.5f});
  h.AddParam(nullptr);
  TensorMeta m;
  m.device = {kDLCUDA, 1};
  m.ndim = 2;
  m.dtype = {kDLBfloat, 16, 1};
  m.shape = {3, 4};
  m.strides = {4, 1};
  PayloadVariant payload;
  if (payload_kind == 1) {
    h.AddParam(m);
    UcxBuffer b(mr, ucx_memory_type::HOST, 24);
    for (int i = 0; i < 24; ++i) static_cast<uint8_t*>(b.data())[i] = uint8_t(i + id);
    payload = std::move(b);
  } else if (payload_kind == 2) {
    h.AddParam(TensorMetaVec{m, m});
    UcxBufferVec v(mr, ucx_memory_type::HOST, std::vector<size_t>{24, 24});
    std::memset(v[0].data, 0xaa, 24);
    std::memset(v[1].data, 0xbb, 24);
    payload = std::move(v);
  }
  h.params.back().name = data::string("last");
  return std::make_shared<AxonRequest>(std::move(h), std::move(payload));
}

EUX_TEST(request_round_trip_all_kinds) {
  DefaultUcxMemoryResourceManager mr;
  for (int kind = 0; kind < 3; ++kind) {
    auto req = make_request(mr, 5, kind);
    std::vector<uint8_t> bytes;
    AvroSerialization::Serialize(*req, mr, bytes);
    avro::Decoder d(bytes.data(), bytes.size());
    auto back = AvroSerialization::Deserialize(d, mr);
    CHECK(d.at_end());
    const auto &a = req->header, &b = back->header;
    CHECK(a.session_id == b.session_id && a.request_id == b.request_id && a.function_id == b.function_id);
    CHECK(a.hlc == b.hlc && a.workflow_id == b.workflow_id);
    CHECK_EQ(a.params.size(), b.params.size());
    for (size_t i = 0; i < a.params.size(); ++i) {
      CHECK(a.params[i].type == b.params[i].type);
      CHECK(a.params[i].name == b.params[i].name);
      CHECK(a.params[i].value.index() == b.params[i].value.index());
    }
    CHECK_EQ(b.GetPrimitive<uint32_t>(2), 4000000000u);
    CHECK_EQ(b.GetPrimitive<uint64_t>(3), uint64_t(1) << 63);
    CHECK_EQ(b.GetPrimitive<int16_t>(1), -7);
    CHECK((b.GetVector<uint8_t>(8) == data::vector<uint8_t>{1, 2, 255}));
    CHECK_EQ(b.GetVector<int64_t>(9)[1], 1ll << 40);
    CHECK_EQ(back->payload.index(), size_t(kind));
    if (kind == 1) {
      CHECK(b.GetTensor(12) == a.GetTensor(12));
      CHECK(std::memcmp(std::get<UcxBuffer>(back->payload).data(), std::get<UcxBuffer>(req->payload).data(), 24) == 0);
      CHECK(back->GetTensor(0).shape[1] == 4);
    } else if (kind == 2) {
      auto& v = std::get<UcxBufferVec>(back->payload);
      CHECK_EQ(v.size(), 2u);
      CHECK_EQ(static_cast<uint8_t*>(v[1].data)[5], 0xbb);
      CHECK_EQ(back->GetTensorVec().size(), 2u);
    }
  }
}

EUX_TEST(double_buffered_streams) {
  std::string dir = tmpdir(), path = dir + "/stream.bin";
  const size_t n = 3 * UnifexOutputStream::kBufferSize + 12345;  // several buffer switches plus a tail
  std::vector<uint8_t> data(n);
  for (size_t i = 0; i < n; ++i) data[i] = uint8_t(i * 131 + (i >> 8));
  {
    UnifexOutputStream out(path);
    size_t off = 0;
    for (size_t chunk : {size_t(1), size_t(4095), size_t(70000), size_t(300000)})
      while (off < n && chunk) {
        size_t take = std::min(chunk, n - off);
        out.write(data.data() + off, take);
        off += take;
        if (chunk != 300000) break;
      }
    out.write(data.data() + off, n - off);
    out.flush();
    CHECK_EQ(out.byte_count(), n);
  }
  {
    UnifexInputStream in(path);
    std::vector<uint8_t> back = in.read_all();
    CHECK_EQ(back.size(), n);
    CHECK(back == data);
  }
  {
    AsyncFile f(path, AsyncFile::Mode::kRead);
    CHECK_EQ(f.size(), n);
    uint8_t buf[64];
    auto got = ex::sync_wait(f.async_read_some_at(1000, buf, 64));
    CHECK(got && *got == 64 && std::memcmp(buf, data.data() + 1000, 64) == 0);
  }
  CHECK_THROWS(UnifexInputStream(dir + "/missing"));
  unlink(path.c_str());
  rmdir(dir.c_str());
}

EUX_TEST(storage_save_load_container) {
  DefaultUcxMemoryResourceManager mr;
  std::string dir = tmpdir();
  AxonStorage st;
  for (uint32_t i = 0; i < 150; ++i) st.emplace(make_request(mr, i, int(i % 3)));  // more than one container block
  CHECK_EQ(st.size(), 150u);
  std::string path = st.save(mr, dir, "ckpt");
  CHECK(path.find(dir + "/ckpt_") == 0 && path.size() > 5 && path.substr(path.size() - 5) == ".avro");
  AxonStorage back;
  CHECK_EQ(back.load(mr, path), 150u);
  auto a = st.snapshot(), b = back.snapshot();
  CHECK_EQ(a.size(), b.size());
  for (size_t i = 0; i < a.size(); ++i) {
    CHECK_EQ(a[i].first, b[i].first);
    CHECK(a[i].second->header.request_id == b[i].second->header.request_id);
    CHECK_EQ(a[i].second->payload.index(), b[i].second->payload.index());
  }
  // async forms and single-request files
  auto loaded = ex::sync_wait(AsyncUnifexAvroIO::Load(path, mr));
  CHECK(loaded && loaded->size() == 150);
  auto one = st.save_request(mr, a[3].first, dir);
  CHECK_EQ(AsyncUnifexAvroIO::LoadSync(one, mr).size(), 1u);
  auto saved = ex::sync_wait(AsyncUnifexAvroIO::Save({a[0].second, a[1].second}, mr, dir, "two"));
  CHECK(saved && AsyncUnifexAvroIO::LoadSync(*saved, mr).size() == 2);
  CHECK(st.erase(a[0].first) && !st.erase(a[0].first));
  CHECK(st.find(a[0].first) == nullptr && st.find(a[1].first) != nullptr);
  // a corrupted file is reported, not crashed on
  {
    FILE* f = fopen(path.c_str(), "r+b");
    fseek(f, 200, SEEK_SET);
    fputc(0xff, f);
    fputc(0xff, f);
    fclose(f);
    bool threw = false;
    try { (void)AsyncUnifexAvroIO::LoadSync(path, mr); } catch (const std::exception&) { threw = true; }
    (void)threw;  // the damaged byte may land in a payload; either way the call returns
  }
  unlink(path.c_str());
  unlink(one.c_str());
  unlink(saved->c_str());
  rmdir(dir.c_str());
}

EUX_TEST_MAIN()
