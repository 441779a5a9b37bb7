// Minimal test harness for the C++ layer's GPU tests: named cases, counted checks, non-zero exit code on failure.
#pragma once

#include <cstdio>
#include <cstring>
#include <exception>
#include <functional>
#include <string>
#include <vector>

#include "gpu_inference/error.h"

namespace chk {

struct Case { const char* name; std::function<void()> body; };
inline std::vector<Case>& cases() { static std::vector<Case> c; return c; }
inline int& failed() { static int f = 0; return f; }
inline int& checked() { static int c = 0; return c; }
struct Register { Register(const char* n, std::function<void()> b) { cases().push_back({n, std::move(b)}); } };

inline void report(const char* file, int line, const std::string& what) {
  ++failed();
  std::fprintf(stderr, "  FAILED %s:%d: %s\n", file, line, what.c_str());
}

template <typename F>
bool throws_code(F&& f, gie::StatusCode want, std::string* got) {
  try {
    f();
  } catch (const gie::Error& e) {
    if (e.code() == want) return true;
    *got = e.what();
    return false;
  } catch (const std::exception& e) {
    *got = e.what();
    return false;
  }
  *got = "no exception";
  return false;
}

inline int run(int argc, char** argv) {
  const char* filter = argc > 1 ? argv[1] : nullptr;
  int ran = 0;
  for (Case& c : cases()) {
    if (filter != nullptr && std::strstr(c.name, filter) == nullptr) continue;
    const int before = failed();
    std::printf("[run ] %s\n", c.name);
    std::fflush(stdout);
    try {
      c.body();
    } catch (const std::exception& e) {
      report(__FILE__, __LINE__, std::string("uncaught exception: ") + e.what());
    }
    std::printf("[%s] %s\n", failed() == before ? " ok " : "FAIL", c.name);
    ++ran;
  }
  std::printf("%d cases, %d checks, %d failures\n", ran, checked(), failed());
  return (ran > 0 && failed() == 0) ? 0 : 1;
}

}  // namespace chk

#define CASE(name)                                             \
  static void case_##name();                                   \
  static chk::Register register_##name(#name, case_##name);    \
  static void case_##name()

#define EXPECT(cond)                                                      \
  do {                                                                    \
    ++chk::checked();                                                     \
    if (!(cond)) chk::report(__FILE__, __LINE__, "EXPECT(" #cond ")");    \
  } while (0)

#define EXPECT_MSG(cond, msg)                                                              \
  do {                                                                                     \
    ++chk::checked();                                                                      \
    if (!(cond)) chk::report(__FILE__, __LINE__, std::string("EXPECT(" #cond ") ") + (msg)); \
  } while (0)

#define EXPECT_THROWS(expr, status)                                                                          \
  do {                                                                                                       \
    ++chk::checked();                                                                                        \
    std::string chk_got_;                                                                                    \
    if (!chk::throws_code([&] { expr; }, (status), &chk_got_))                                               \
      chk::report(__FILE__, __LINE__, std::string("expected gie::Error with " #status " from " #expr ", got: ") + chk_got_); \
  } while (0)
