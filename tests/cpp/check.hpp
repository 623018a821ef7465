// Minimal assert runner (googletest is not installable here): CHECK / CHECK_EQ count failures, report file:line.
#pragma once
#include <cstdio>
#include <iostream>
#include <sstream>
#include <string>
#include <vector>

namespace tiny_test {
inline int &failures() { static int f = 0; return f; }
inline int &checks() { static int c = 0; return c; }
struct Case { const char *name; void (*fn)(); };
inline std::vector<Case> &cases() { static std::vector<Case> c; return c; }
struct Registrar { Registrar(const char *n, void (*f)()) { cases().push_back({n, f}); } };
inline int run_all(const char *filter = nullptr) {
    for (auto &c : cases()) {
        if (filter && !std::string(c.name).find(filter) == 0 && std::string(c.name).find(filter) == std::string::npos) continue;
        const int before = failures();
        c.fn();
        std::printf("[%s] %s\n", failures() == before ? " OK " : "FAIL", c.name);
    }
    std::printf("%d checks, %d failures\n", checks(), failures());
    return failures() ? 1 : 0;
}
}  // namespace tiny_test

#define TEST_CASE(name) static void name(); static tiny_test::Registrar reg_##name(#name, name); static void name()
#define CHECK(cond) do { ++tiny_test::checks(); if (!(cond)) { ++tiny_test::failures(); std::printf("  %s:%d: CHECK(%s) failed\n", __FILE__, __LINE__, #cond); } } while (0)
#define CHECK_EQ(a, b) do { ++tiny_test::checks(); if (!((a) == (b))) { ++tiny_test::failures(); std::printf("  %s:%d: CHECK_EQ(%s, %s) failed\n", __FILE__, __LINE__, #a, #b); } } while (0)
