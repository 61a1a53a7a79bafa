// Host-side sweep of the scalar building blocks the kernels are made of (gefen_b200/csrc/quant_core.h),
// compiled by g++ for the CPU test-suite: the table-driven quantiser and the threshold form must agree
// with the reference rule for EVERY float in [-1, 1] (exhaustive mode) or for a dense sample, and the
// two-FMA division must equal the IEEE quotient.
//
//   quant_core_sweep <codebook.f32> <mode: full|sample> -> prints "mismatch_lut mismatch_thr slow_hits div_mismatch checked"
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>
#include <random>
#include "../../gefen_b200/csrc/quant_core.h"

using namespace gefen;

int main(int argc, char** argv) {
    if (argc < 3) return 2;
    FILE* f = fopen(argv[1], "rb");
    if (!f) return 2;
    std::vector<float> cb(256);
    const int k = static_cast<int>(fread(cb.data(), 4, 256, f));
    fclose(f);
    if (k < 1) return 2;
    const bool full = strcmp(argv[2], "full") == 0;

    std::vector<float> pad(256), thr(256);
    for (int i = 0; i < 256; ++i) pad[i] = cb[i < k ? i : k - 1];
    std::vector<int> tcell(256);
    for (int i = 0; i < 256; ++i) {
        thr[i] = (i < k - 1) ? entry_threshold(i, pad.data(), k) : INFINITY;
        tcell[i] = lut_threshold_cell(thr[i]);
    }
    std::vector<uint32_t> lut(kLutBytes / 4, 0u);
    for (int c = 0; c <= kLutCells; ++c)
        lut_build_cell(c, tcell.data(), thr.data(), k - 1, pad[k - 1], &lut[2 * c], &lut[2 * c + 1]);
    const unsigned char* lut_bytes = reinterpret_cast<const unsigned char*>(lut.data());

    unsigned long long bad_lut = 0, bad_thr = 0, slow_hits = 0, checked = 0;
    const uint32_t lo = float_to_ordered(-1.0f), hi = float_to_ordered(1.0f);
    const uint32_t stride = full ? 1u : 1021u;
#pragma omp parallel for reduction(+ : bad_lut, bad_thr, slow_hits, checked) schedule(static)
    for (long long o = lo; o <= static_cast<long long>(hi); o += stride) {
        const float x = ordered_to_float(static_cast<uint32_t>(o));
        const int want = nearest_entry_reference(x, pad.data(), k);
        bool slow;
        int got = lut_query(x, lut_bytes, &slow);
        if (slow) { ++slow_hits; got = entry_exact(x, thr.data(), pad.data(), k); }
        if (got != want) ++bad_lut;
        if (entry_exact(x, thr.data(), pad.data(), k) != want) ++bad_thr;
        ++checked;
    }
    // special values through the threshold form
    const float specials[] = {NAN, INFINITY, -INFINITY, 2.0f, -2.0f, 0.0f, -0.0f};
    for (float x : specials)
        if (entry_exact(x, thr.data(), pad.data(), k) != nearest_entry_reference(x, pad.data(), k)) ++bad_thr;

    // division: a / b for |a| <= b, b in the supported range
    unsigned long long bad_div = 0;
    std::mt19937_64 rng(1234);
    std::uniform_real_distribution<float> ua(-1.0f, 1.0f);
    std::uniform_real_distribution<float> ue(-60.0f, 60.0f);
    const long long n_div = full ? 400000000LL : 20000000LL;
    std::vector<float> bs, as;
    for (int i = 0; i < 4096; ++i) {
        float b = exp2f(ue(rng)) * (1.0f + fabsf(ua(rng)));
        if (i % 7 == 0) { uint32_t u; memcpy(&u, &b, 4); u |= 0x007fffffu; memcpy(&b, &u, 4); }  // mantissa all ones
        if (i % 11 == 0) { uint32_t u; memcpy(&u, &b, 4); u &= 0xff800000u; memcpy(&b, &u, 4); } // power of two
        bs.push_back(b);
    }
#pragma omp parallel for reduction(+ : bad_div) schedule(static)
    for (long long i = 0; i < n_div; ++i) {
        std::mt19937_64 r(static_cast<unsigned long long>(i) * 2654435761ULL + 17);
        const float b = bs[r() & 4095];
        if (!div_range_ok(b)) continue;
        float a;
        const unsigned long long pick = r();
        if ((pick & 15) == 0) a = b; else if ((pick & 15) == 1) a = -b;
        else a = b * (static_cast<float>(static_cast<double>(r() >> 11) * (1.0 / 9007199254740992.0)) * 2.0f - 1.0f);
        if (fabsf(a) > b) a = b;
        const float rb = 1.0f / b;
        const float q = div_by_block_constant(a, b, rb);
        const float want = a / b;
        if (!(q == want) ) ++bad_div;
    }
    printf("%llu %llu %llu %llu %llu\n", bad_lut, bad_thr, slow_hits, bad_div, checked);
    return 0;
}
