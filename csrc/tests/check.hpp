// Minimal test harness for the C++ unit tests (no external framework is available).
#pragma once
#include <cstdio>
#include <cstdlib>
#include <exception>
#include <functional>
#include <string>
#include <vector>

namespace eux::test {
struct registry {
  static std::vector<std::pair<std::string, std::function<void()>>>& tests() {
    static std::vector<std::pair<std::string, std::function<void()>>> t;
    return t;
  }
};
struct reg {
  reg(const char* name, std::function<void()> f) { registry::tests().emplace_back(name, std::move(f)); }
};
struct failure : std::exception {
  std::string msg;
  explicit failure(std::string m) : msg(std::move(m)) {}
  const char* what() const noexcept override { return msg.c_str(); }
};
inline int run_all(int argc, char** argv) {
  std::string filter = argc > 1 ? argv[1] : "";
  int failed = 0, ran = 0;
  for (auto& [name, fn] : registry::tests()) {
    if (!filter.empty() && name.find(filter) == std::string::npos) continue;
    ++ran;
    try {
      fn();
      std::printf("[ OK ] %s\n", name.c_str());
    } catch (const std::exception& e) {
      ++failed;
      std::printf("[FAIL] %s: %s\n", name.c_str(), e.what());
    }
    std::fflush(stdout);
  }
  std::printf("%d tests, %d failed\n", ran, failed);
  return failed ? 1 : 0;
}
}  // namespace eux::test

#define EUX_TEST(name)                                            \
  static void eux_test_##name();                                  \
  static ::eux::test::reg eux_reg_##name(#name, eux_test_##name); \
  static void eux_test_##name()
#define EUX_STR2(x) #x
#define EUX_STR(x) EUX_STR2(x)
#define CHECK(cond)                                                                              \
  do {                                                                                           \
    if (!(cond)) throw ::eux::test::failure(__FILE__ ":" EUX_STR(__LINE__) ": CHECK(" #cond ")"); \
  } while (0)
#define CHECK_EQ(a, b) CHECK((a) == (b))
#define CHECK_THROWS(expr)                                                                                  \
  do {                                                                                                      \
    bool threw_ = false;                                                                                    \
    try {                                                                                                   \
      (void)(expr);                                                                                         \
    } catch (...) {                                                                                         \
      threw_ = true;                                                                                        \
    }                                                                                                       \
    if (!threw_) throw ::eux::test::failure(__FILE__ ":" EUX_STR(__LINE__) ": expected a throw: " #expr); \
  } while (0)
#define EUX_TEST_MAIN() \
  int main(int argc, char** argv) { return ::eux::test::run_all(argc, argv); }
