// Stand-in for the macOS header that src/core/thread_pool.cpp includes: the lookup always
// fails, so the pool falls back to std::thread::hardware_concurrency().
#pragma once
#include <cstddef>
inline int sysctlbyname(const char*, void*, size_t*, void*, size_t) { return -1; }
