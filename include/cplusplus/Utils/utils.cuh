// Index helpers with the names upstream's sources use (include/cplusplus/Utils/utils.cuh:14-44 there),
// kept so that upstream code keeps compiling against this tree.  Unlike upstream they widen to 64 bits:
// K/V of the long-context configuration hold 2^30 elements, which overflows int arithmetic in bytes.
#pragma once

#include <cstdint>

#if defined(__CUDACC__)
#define CLLO_HD __host__ __device__
#else
#define CLLO_HD
#endif

CLLO_HD constexpr int CEIL_DIV(int numerator, int denominator) {
    return numerator / denominator + (numerator % denominator != 0 ? 1 : 0);
}

CLLO_HD constexpr std::int64_t GET_1D_INDEX_FROM_3D(std::int64_t a, std::int64_t b, std::int64_t c, std::int64_t nb,
                                                    std::int64_t nc) {
    return (a * nb + b) * nc + c;
}

CLLO_HD constexpr std::int64_t GET_1D_INDEX_FROM_4D(std::int64_t a, std::int64_t b, std::int64_t c, std::int64_t d,
                                                    std::int64_t nb, std::int64_t nc, std::int64_t nd) {
    return ((a * nb + b) * nc + c) * nd + d;
}
