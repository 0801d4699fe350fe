// Minimal native test harness: TEST(name) { ... } registers a case; CHECK / CHECK_EQ /
// CHECK_NEAR / CHECK_THROWS record failures without aborting the case; the runner prints one
// line per case and returns the number of failed cases.
#pragma once
#include <cmath>
#include <cstdio>
#include <functional>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

namespace obtest {

struct Case {
  const char* name;
  std::function<void()> body;
};

inline std::vector<Case>& registry() {
  static std::vector<Case> cases;
  return cases;
}
inline int& failures_in_case() {
  static int n = 0;
  return n;
}
inline void fail(const char* file, int line, const std::string& what) {
  ++failures_in_case();
  std::printf("    %s:%d: %s\n", file, line, what.c_str());
}

struct Registrar {
  Registrar(const char* name, std::function<void()> body) { registry().push_back({name, std::move(body)}); }
};

inline int run_all(const char* filter) {
  int failed = 0, ran = 0;
  for (const Case& c : registry()) {
    if (filter && std::string(c.name).find(filter) == std::string::npos) continue;
    failures_in_case() = 0;
    try {
      c.body();
    } catch (const std::exception& e) {
      fail("<case>", 0, std::string("unexpected exception: ") + e.what());
    } catch (...) {
      fail("<case>", 0, "unexpected non-standard exception");
    }
    ++ran;
    if (failures_in_case()) ++failed;
    std::printf("[%s] %s\n", failures_in_case() ? "FAILED" : "  OK  ", c.name);
  }
  std::printf("native tests: %d run, %d failed\n", ran, failed);
  return failed;
}

}  // namespace obtest

#define OBT_CAT2(a, b) a##b
#define OBT_CAT(a, b) OBT_CAT2(a, b)
#define TEST(name)                                                              \
  static void OBT_CAT(obt_body_, name)();                                       \
  static ::obtest::Registrar OBT_CAT(obt_reg_, name)(#name, OBT_CAT(obt_body_, name)); \
  static void OBT_CAT(obt_body_, name)()

#define CHECK(cond)                                                   \
  do {                                                                \
    if (!(cond)) ::obtest::fail(__FILE__, __LINE__, "CHECK(" #cond ")"); \
  } while (0)
#define CHECK_EQ(a, b)                                                                   \
  do {                                                                                   \
    const auto obt_a = (a);                                                              \
    const auto obt_b = (b);                                                              \
    if (!(obt_a == obt_b)) {                                                             \
      std::ostringstream obt_os;                                                         \
      obt_os << "CHECK_EQ(" #a ", " #b "): " << obt_a << " vs " << obt_b;                 \
      ::obtest::fail(__FILE__, __LINE__, obt_os.str());                                  \
    }                                                                                    \
  } while (0)
#define CHECK_NEAR(a, b, tol)                                                            \
  do {                                                                                   \
    const double obt_a = static_cast<double>(a), obt_b = static_cast<double>(b);         \
    if (!(std::fabs(obt_a - obt_b) <= (tol))) {                                          \
      std::ostringstream obt_os;                                                         \
      obt_os << "CHECK_NEAR(" #a ", " #b "): " << obt_a << " vs " << obt_b;               \
      ::obtest::fail(__FILE__, __LINE__, obt_os.str());                                  \
    }                                                                                    \
  } while (0)
#define CHECK_THROWS(expr)                                                               \
  do {                                                                                   \
    bool obt_threw = false;                                                              \
    try { (void)(expr); } catch (const std::exception&) { obt_threw = true; }            \
    if (!obt_threw) ::obtest::fail(__FILE__, __LINE__, "CHECK_THROWS(" #expr ")");       \
  } while (0)
#define CHECK_THROWS_WITH(expr, text)                                                    \
  do {                                                                                   \
    std::string obt_msg;                                                                 \
    bool obt_threw = false;                                                              \
    try { (void)(expr); } catch (const std::exception& e) { obt_threw = true; obt_msg = e.what(); } \
    if (!obt_threw || obt_msg.find(text) == std::string::npos)                           \
      ::obtest::fail(__FILE__, __LINE__, std::string("CHECK_THROWS_WITH(" #expr "): got '") + obt_msg + "'"); \
  } while (0)
