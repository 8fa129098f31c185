// Minimal host-only test harness: TEST(name) registers a function, EXPECT records failures,
// the runner prints one "[ OK ]/[FAIL] name" line per test and exits 1 on any failure.
// No GPU, no NCCL: everything device- or network-facing is replaced by the fakes in fakes.h
// (the reference reaches the same isolation with link-seam fakes, tests/coccl-tests/src/Makefile:243-502).
#pragma once
#include <stdio.h>
#include <string>
#include <vector>

namespace host_test {
struct Case { const char* name; void (*fn)(); };
std::vector<Case>& registry();
extern int gFailures;
struct Registrar { Registrar(const char* n, void (*f)()) { registry().push_back({n, f}); } };
}  // namespace host_test

#define TEST(name)                                                        \
  static void test_##name();                                              \
  static host_test::Registrar registrar_##name(#name, &test_##name);      \
  static void test_##name()

#define EXPECT(cond)                                                                      \
  do {                                                                                    \
    if (!(cond)) {                                                                        \
      ++host_test::gFailures;                                                             \
      fprintf(stderr, "  EXPECT failed: %s (%s:%d)\n", #cond, __FILE__, __LINE__);        \
    }                                                                                     \
  } while (0)
#define EXPECT_EQ(a, b)                                                                                   \
  do {                                                                                                    \
    auto va_ = (a);                                                                                       \
    auto vb_ = (b);                                                                                       \
    if (!(va_ == vb_)) {                                                                                  \
      ++host_test::gFailures;                                                                             \
      fprintf(stderr, "  EXPECT_EQ failed: %s == %s (%lld vs %lld) (%s:%d)\n", #a, #b, (long long)va_,    \
              (long long)vb_, __FILE__, __LINE__);                                                        \
    }                                                                                                     \
  } while (0)
