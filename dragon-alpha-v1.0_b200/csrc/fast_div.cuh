// Division of x < 2^31 by a positive constant d as a multiplication: floor(x / d) == (x * m) >> s with
// s = 31 + ceil(log2 d), m = floor(2^s / d) + 1 (the error term x * (m * d - 2^s) stays below 2^s).  The HBM-bound
// gather kernels spend a few loads per element; a handful of hardware divisions per element would cost more than
// the loads.
#pragma once

namespace alpha {

struct FastDiv {
    unsigned long long m;
    unsigned d;
    int s;
    __host__ __device__ unsigned div(unsigned x) const { return static_cast<unsigned>((static_cast<unsigned long long>(x) * m) >> s); }
    __host__ __device__ void divmod(unsigned x, unsigned& q, unsigned& r) const { q = div(x); r = x - q * d; }
};

inline FastDiv fast_div(int d_)
{
    const unsigned d = static_cast<unsigned>(d_);
    int b = 0;
    while ((1ull << b) < d) ++b;
    FastDiv f;
    f.d = d; f.s = 31 + b;
    f.m = (1ull << f.s) / d + 1;
    return f;
}

}  // namespace alpha
