// Value types of the RPC wire model. In memory they are ordinary standard
// containers; their serialised form is the cista "offset" image that the
// reference puts on the wire (see utils/cista_serialize_helper.hpp), so the
// names follow cista's: data::string, data::vector<T>, data::variant, strong<T>.
#pragma once

#include <cstddef>
#include <cstdint>
#include <functional>
#include <string>
#include <string_view>
#include <type_traits>
#include <variant>
#include <vector>

namespace eux::rpc {

namespace data {

// std::string with cista's accessors
class string : public std::string {
 public:
  using std::string::string;
  string() = default;
  string(const std::string& s) : std::string(s) {}
  string(std::string&& s) : std::string(std::move(s)) {}
  string(std::string_view s) : std::string(s) {}
  const std::string& str() const { return *this; }
  std::string_view view() const { return std::string_view(data(), size()); }
};

// One byte per element on the wire; std::vector<bool> is a bit set, so bools are wrapped.
struct bool_t {
  bool value = false;
  bool_t() = default;
  bool_t(bool b) : value(b) {}
  operator bool() const { return value; }
};
static_assert(sizeof(bool_t) == 1);

template <class T>
using vector = std::vector<std::conditional_t<std::is_same_v<T, bool>, bool_t, T>>;

template <class... T>
using variant = std::variant<T...>;

}  // namespace data

// A distinct integer type (cista::strong): the value is the public member v_.
template <class T, class Tag>
struct strong {
  using value_t = T;
  constexpr strong() = default;
  explicit constexpr strong(T v) : v_(v) {}
  constexpr T value() const { return v_; }
  friend constexpr bool operator==(const strong& a, const strong& b) { return a.v_ == b.v_; }
  friend constexpr auto operator<=>(const strong& a, const strong& b) { return a.v_ <=> b.v_; }
  strong& operator++() {
    ++v_;
    return *this;
  }
  T v_{};
};

using byte_buf = std::vector<std::uint8_t>;

}  // namespace eux::rpc

namespace std {
template <class T, class Tag>
struct hash<eux::rpc::strong<T, Tag>> {
  size_t operator()(const eux::rpc::strong<T, Tag>& s) const noexcept { return std::hash<T>{}(s.v_); }
};
template <>
struct hash<eux::rpc::data::string> {
  size_t operator()(const eux::rpc::data::string& s) const noexcept { return std::hash<std::string>{}(s); }
};
}  // namespace std
