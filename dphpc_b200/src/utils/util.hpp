// Output switches of the benchmark driver: FILE_DUMP prints the CSV rows, DEBUG_OUT the
// chatty progress lines (off by default), as in the reference's src/utils/util.hpp:5-20.
#pragma once
#include <iostream>

#ifndef SDDMM_NO_DUMP
#define FILE_DUMP(x) do { std::cout << x; } while (0)
#else
#define FILE_DUMP(x) do { } while (0)
#endif

#ifdef SDDMM_DEBUG
#define DEBUG_OUT(x) do { std::cerr << x; } while (0)
#else
#define DEBUG_OUT(x) do { } while (0)
#endif
