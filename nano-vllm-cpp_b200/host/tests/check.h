// Tiny check harness for the C++ tests of the operator layer (no test framework is available).
#pragma once

#include <cmath>
#include <cstdio>
#include <exception>
#include <functional>
#include <string>
#include <vector>

namespace check {

struct Registry {
    std::vector<std::pair<std::string, std::function<void()>>> tests;
    int failures = 0;
    static Registry& get() {
        static Registry r;
        return r;
    }
};

struct Registrar {
    Registrar(const char* name, std::function<void()> fn) { Registry::get().tests.emplace_back(name, std::move(fn)); }
};

inline void fail(const char* file, int line, const std::string& what) {
    std::fprintf(stderr, "  FAIL %s:%d: %s\n", file, line, what.c_str());
    ++Registry::get().failures;
}

inline int run_all() {
    Registry& r = Registry::get();
    int failed_tests = 0;
    for (auto& t : r.tests) {
        const int before = r.failures;
        try {
            t.second();
        } catch (const std::exception& e) {
            fail(t.first.c_str(), 0, std::string("unexpected exception: ") + e.what());
        }
        const bool ok = r.failures == before;
        std::printf("[%s] %s\n", ok ? " OK " : "FAIL", t.first.c_str());
        if (!ok) ++failed_tests;
    }
    std::printf("%zu tests, %d failed\n", r.tests.size(), failed_tests);
    return failed_tests == 0 ? 0 : 1;
}

}  // namespace check

#define TEST_CASE(name)                                             \
    static void test_##name();                                      \
    static check::Registrar registrar_##name(#name, test_##name);   \
    static void test_##name()

#define CHECK(cond)                                                  \
    do {                                                             \
        if (!(cond)) check::fail(__FILE__, __LINE__, #cond);         \
    } while (0)

#define CHECK_EQ(a, b)                                                                        \
    do {                                                                                      \
        if (!((a) == (b))) check::fail(__FILE__, __LINE__, std::string(#a " == " #b));        \
    } while (0)

#define CHECK_NEAR(a, b, tol)                                                                              \
    do {                                                                                                   \
        const double va_ = (a), vb_ = (b);                                                                 \
        if (!(std::fabs(va_ - vb_) <= (tol)))                                                              \
            check::fail(__FILE__, __LINE__, std::string(#a " ~ " #b ": ") + std::to_string(va_) + " vs " + \
                                                std::to_string(vb_));                                      \
    } while (0)

#define CHECK_THROWS(expr, ExceptionType)                                                    \
    do {                                                                                     \
        bool caught_ = false;                                                                \
        try {                                                                                \
            expr;                                                                            \
        } catch (const ExceptionType&) {                                                     \
            caught_ = true;                                                                  \
        } catch (...) {                                                                      \
        }                                                                                    \
        if (!caught_) check::fail(__FILE__, __LINE__, #expr " should throw " #ExceptionType); \
    } while (0)
