// Host-side check of the multiply-shift division used by the gather kernels (csrc/fast_div.cuh):
// for every divisor d in a range and for the dividends where an error would first show (multiples of d and
// their neighbours, up to 2^31 - 1) the quotient and remainder must equal x / d and x % d.
#include <cstdio>
#include <cstdlib>
#include "../dragon-alpha-v1.0_b200/csrc/fast_div.cuh"

static long long check(unsigned d, unsigned x)
{
    const alpha::FastDiv f = alpha::fast_div(static_cast<int>(d));
    unsigned q, r;
    f.divmod(x, q, r);
    return (q == x / d && r == x % d) ? 0 : 1;
}

int main(int argc, char** argv)
{
    const unsigned dmax = argc > 1 ? static_cast<unsigned>(atoi(argv[1])) : 5000u;
    const unsigned top = 2147483647u;
    long long bad = 0, n = 0;
    unsigned long long seed = 0x9E3779B97F4A7C15ull;
    for (unsigned d = 1; d <= dmax; ++d) {
        const unsigned kmax = top / d;
        const unsigned ks[] = {0u, 1u, 2u, kmax / 3, kmax / 2, kmax - 1, kmax};
        for (unsigned k : ks)
            for (int off = -2; off <= 2; ++off) {
                const long long x = static_cast<long long>(k) * d + off;
                if (x < 0 || x > top) continue;
                bad += check(d, static_cast<unsigned>(x)); ++n;
            }
        bad += check(d, top); ++n;
        for (int i = 0; i < 64; ++i) {
            seed = seed * 6364136223846793005ull + 1442695040888963407ull;
            bad += check(d, static_cast<unsigned>(seed >> 33)); ++n;   // 31-bit dividends
        }
    }
    // large divisors too (tensor extents)
    for (unsigned d : {65535u, 65536u, 65537u, 1000003u, 16777216u, 1073741823u, 1073741824u, 2147483647u})
        for (unsigned x : {0u, d - 1, d, d + 1 > top ? top : d + 1, top - 1, top}) { bad += check(d, x); ++n; }
    printf("%lld checks, %lld wrong\n", n, bad);
    return bad ? 1 : 0;
}
