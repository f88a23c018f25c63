// Status codes of the transport layer and their std::error_code category "UCX".
// The numeric values are the ones OpenUCX uses for ucs_status_t, because they
// travel in completion entries and in RpcStatus on the wire
// (reference: ucx_context/ucx_status.hpp:35-150 maps ucs_status_t the same way;
// UCS_OK and UCS_INPROGRESS both mean "no error").
#pragma once

#include <string>
#include <system_error>

namespace eux::ucxx {

enum ucs_status_t : int {
  UCS_OK = 0,
  UCS_INPROGRESS = 1,
  UCS_ERR_NO_MESSAGE = -1,
  UCS_ERR_NO_RESOURCE = -2,
  UCS_ERR_IO_ERROR = -3,
  UCS_ERR_NO_MEMORY = -4,
  UCS_ERR_INVALID_PARAM = -5,
  UCS_ERR_UNREACHABLE = -6,
  UCS_ERR_INVALID_ADDR = -7,
  UCS_ERR_NOT_IMPLEMENTED = -8,
  UCS_ERR_MESSAGE_TRUNCATED = -9,
  UCS_ERR_NO_PROGRESS = -10,
  UCS_ERR_BUFFER_TOO_SMALL = -11,
  UCS_ERR_NO_ELEM = -12,
  UCS_ERR_SOME_CONNECTS_FAILED = -13,
  UCS_ERR_NO_DEVICE = -14,
  UCS_ERR_BUSY = -15,
  UCS_ERR_CANCELED = -16,
  UCS_ERR_SHMEM_SEGMENT = -17,
  UCS_ERR_ALREADY_EXISTS = -18,
  UCS_ERR_OUT_OF_RANGE = -19,
  UCS_ERR_TIMED_OUT = -20,
  UCS_ERR_EXCEEDS_LIMIT = -21,
  UCS_ERR_UNSUPPORTED = -22,
  UCS_ERR_REJECTED = -23,
  UCS_ERR_NOT_CONNECTED = -24,
  UCS_ERR_CONNECTION_RESET = -25,
  UCS_ERR_ENDPOINT_TIMEOUT = -80,
  UCS_ERR_LAST = -100
};

inline const char* ucs_status_string(int s) noexcept {
  switch (s) {
    case UCS_OK: return "Success";
    case UCS_INPROGRESS: return "Operation in progress";
    case UCS_ERR_NO_MESSAGE: return "No pending message";
    case UCS_ERR_NO_RESOURCE: return "No resources are available to initiate the operation";
    case UCS_ERR_IO_ERROR: return "Input/output error";
    case UCS_ERR_NO_MEMORY: return "Out of memory";
    case UCS_ERR_INVALID_PARAM: return "Invalid parameter";
    case UCS_ERR_UNREACHABLE: return "Destination is unreachable";
    case UCS_ERR_INVALID_ADDR: return "Address not valid";
    case UCS_ERR_NOT_IMPLEMENTED: return "Function not implemented";
    case UCS_ERR_MESSAGE_TRUNCATED: return "Message truncated";
    case UCS_ERR_NO_PROGRESS: return "No progress";
    case UCS_ERR_BUFFER_TOO_SMALL: return "Provided buffer is too small";
    case UCS_ERR_NO_ELEM: return "No such element";
    case UCS_ERR_SOME_CONNECTS_FAILED: return "Failed to connect some of the requested endpoints";
    case UCS_ERR_NO_DEVICE: return "No such device";
    case UCS_ERR_BUSY: return "Device is busy";
    case UCS_ERR_CANCELED: return "Request canceled";
    case UCS_ERR_SHMEM_SEGMENT: return "Shared memory error";
    case UCS_ERR_ALREADY_EXISTS: return "Element already exists";
    case UCS_ERR_OUT_OF_RANGE: return "Index out of range";
    case UCS_ERR_TIMED_OUT: return "Operation timed out";
    case UCS_ERR_EXCEEDS_LIMIT: return "User-defined limit was reached";
    case UCS_ERR_UNSUPPORTED: return "Unsupported operation";
    case UCS_ERR_REJECTED: return "Operation rejected by remote peer";
    case UCS_ERR_NOT_CONNECTED: return "Endpoint is not connected";
    case UCS_ERR_CONNECTION_RESET: return "Connection reset by remote peer";
    case UCS_ERR_ENDPOINT_TIMEOUT: return "Endpoint timeout";
    default: return "Unknown error";
  }
}

class ucx_error_category_t final : public std::error_category {
 public:
  const char* name() const noexcept override { return "UCX"; }
  std::string message(int ev) const override { return ucs_status_string(ev); }
  std::error_condition default_error_condition(int ev) const noexcept override {
    if (ev == UCS_OK || ev == UCS_INPROGRESS) return std::error_condition(0, std::generic_category());
    switch (ev) {
      case UCS_ERR_NO_MEMORY: return std::errc::not_enough_memory;
      case UCS_ERR_INVALID_PARAM: return std::errc::invalid_argument;
      case UCS_ERR_UNREACHABLE: return std::errc::host_unreachable;
      case UCS_ERR_TIMED_OUT: case UCS_ERR_ENDPOINT_TIMEOUT: return std::errc::timed_out;
      case UCS_ERR_CANCELED: return std::errc::operation_canceled;
      case UCS_ERR_NOT_CONNECTED: return std::errc::not_connected;
      case UCS_ERR_CONNECTION_RESET: return std::errc::connection_reset;
      case UCS_ERR_BUSY: return std::errc::device_or_resource_busy;
      case UCS_ERR_NOT_IMPLEMENTED: case UCS_ERR_UNSUPPORTED: return std::errc::not_supported;
      default: return std::error_condition(ev, *this);
    }
  }
};

inline const std::error_category& ucx_category() noexcept {
  static const ucx_error_category_t cat;
  return cat;
}
inline std::error_code make_error_code(ucs_status_t s) noexcept { return {static_cast<int>(s), ucx_category()}; }
inline std::error_code make_ucx_error(int s) noexcept { return {s, ucx_category()}; }
inline bool ucs_is_error(int s) noexcept { return s < 0; }

}  // namespace eux::ucxx

namespace std {
template <>
struct is_error_code_enum<eux::ucxx::ucs_status_t> : true_type {};
}  // namespace std
