#include <string.h>

#include "host_test.h"

namespace host_test {
std::vector<Case>& registry() {
  static std::vector<Case> r;
  return r;
}
int gFailures = 0;
}  // namespace host_test

int main(int argc, char** argv) {
  const char* filter = argc > 1 ? argv[1] : nullptr;
  int failed = 0, ran = 0;
  for (const auto& c : host_test::registry()) {
    if (filter && !strstr(c.name, filter)) continue;
    const int before = host_test::gFailures;
    c.fn();
    ++ran;
    const bool ok = host_test::gFailures == before;
    printf("[%s] %s\n", ok ? " OK " : "FAIL", c.name);
    if (!ok) ++failed;
  }
  printf("%d tests, %d failed\n", ran, failed);
  return failed ? 1 : 0;
}
