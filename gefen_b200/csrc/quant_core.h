// Scalar building blocks shared by every Gefen kernel: the nearest-codebook-entry rule,
// its exact threshold form, the uniform-grid lookup table that answers it in one shared-memory
// read, and an exactly rounded division by a per-block constant.
//
// Everything here is `__host__ __device__` so that the same code can be compiled by g++ and
// swept exhaustively on a CPU (tests do that); the product only ever runs it on the GPU.
//
// Reference semantics being reproduced (reference: kernels/automatic_gefen_fused_kernel.cu:59-90):
//   lower_bound over the sorted codebook, then the closer of the two neighbours, the LEFT one on
//   a tie of the two float distances.
#pragma once

#include <stdint.h>
#include <math.h>

#if defined(__CUDACC__)
#define GEFEN_HD __host__ __device__ __forceinline__
#else
#define GEFEN_HD static inline
#endif

namespace gefen {

constexpr int kMaxCodebook = 256;          // reference: at most 256 entries (uint8 codes)
constexpr int kLutCells = 4096;            // cells over [-1, 1); one more cell for x == 1
constexpr int kLutBytes = 32784;           // 4097 entries of 8 bytes, padded to a multiple of 16
constexpr uint32_t kLutSlowBit = 0x80000000u;    // cell cannot be decided by one comparison

struct alignas(8) uint2v { uint32_t x, y; };   // 8-byte table entry, read with one 64-bit load

// ---------------------------------------------------------------------------------------------
// The reference rule, verbatim in behaviour. NaN maps to entry 0 (every comparison is false).
GEFEN_HD int nearest_entry_reference(float x, const float* cb, int k) {
    int lo = 0, hi = k;
    while (lo < hi) {
        const int mid = lo + (hi - lo) / 2;
        if (cb[mid] < x) lo = mid + 1; else hi = mid;
    }
    int r = lo;
    if (r >= k) r = k - 1;
    int l = r - 1;
    if (l < 0) l = 0;
    const float dl = fabsf(x - cb[l]);
    const float dr = fabsf(x - cb[r]);
    return dl <= dr ? l : r;
}

// Order-preserving map between floats and unsigned integers (NaN excluded).
GEFEN_HD uint32_t float_to_ordered(float f) {
    union { float f; uint32_t u; } c; c.f = f;
    return (c.u & 0x80000000u) ? ~c.u : (c.u | 0x80000000u);
}
GEFEN_HD float ordered_to_float(uint32_t o) {
    union { float f; uint32_t u; } c;
    c.u = (o & 0x80000000u) ? (o & 0x7FFFFFFFu) : ~o;
    return c.f;
}

// For x up to the last codebook entry the rule above is a non-decreasing step function of x
// (fl(x-a) grows with x, fl(b-x) shrinks), so there it is fully described by k-1 thresholds:
// entry(x) = #{ i : T_i < x }. T_i is the largest float <= cb[k-1] whose entry is <= i, found by
// bisection over the ordered float keys; +inf when no x <= cb[k-1] gets past entry i.
// Above the last entry the rule is NOT monotone (both distances can round to the same float, and
// the tie goes left), so that range is answered directly, see entry_exact.
GEFEN_HD float entry_threshold(int i, const float* cb, int k) {
    uint32_t lo = float_to_ordered(-INFINITY);   // entry(-inf) == 0 <= i always
    uint32_t hi = float_to_ordered(cb[k - 1]);
    if (nearest_entry_reference(cb[k - 1], cb, k) <= i) return INFINITY;
    while (hi - lo > 1u) {
        const uint32_t mid = lo + ((hi - lo) >> 1);
        if (nearest_entry_reference(ordered_to_float(mid), cb, k) <= i) lo = mid; else hi = mid;
    }
    return ordered_to_float(lo);
}

// Count of thresholds strictly below x. thr must hold 256 floats, the unused tail = +inf.
// Equals the reference rule for every float x <= cb[k-1], NaN included (-> 0).
GEFEN_HD int entry_by_thresholds(float x, const float* thr) {
    int pos = 0;
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
    for (int s = 128; s > 0; s >>= 1) {
        if (thr[pos + s - 1] < x) pos += s;
    }
    // pos counts thresholds among the first 255; slot 255 is always +inf padding.
    return pos;
}

// The reference rule for every float, through the thresholds. `cb` is the codebook padded to 256
// entries with its last value, `k` its true size.
GEFEN_HD int entry_exact(float x, const float* thr, const float* cb, int k) {
    if (x > cb[k - 1]) {   // lower_bound == k: neighbours k-2 and k-1, left on ties
        const int l = k >= 2 ? k - 2 : 0;
        return fabsf(x - cb[l]) <= fabsf(x - cb[k - 1]) ? l : k - 1;
    }
    return entry_by_thresholds(x, thr);
}

// ---------------------------------------------------------------------------------------------
// Uniform-grid lookup table over x in [-1, 1]: 4096 cells of width 2^-11 (one more for x == 1),
// the width of one bin of the 4096-bin histogram the codebook is fitted to, so that codebooks from
// that fit put at most one threshold in almost every cell.
// Cell of x: the integer part of fma(x, 16384, magic) keeps round(x * 16384) + 16384 in its low
// mantissa bits; masking the low three bits gives the BYTE offset of the 8-byte table entry. The
// map is monotone in x, which is all the table needs: every threshold in a lower cell is below x,
// every threshold in a higher cell is above it, and the one threshold that may share x's cell is
// compared exactly in float. entry(x) = below(cell) + (x > threshold(cell)).
// Entry layout: word 0 = float bits of the cell's threshold (+inf if none), word 1 = number of
// thresholds below the cell, bit 31 set when the cell cannot be decided this way (two or more
// thresholds inside, or values above the last codebook entry): values in such cells go through
// entry_exact.
GEFEN_HD uint32_t lut_byte_offset(float x) {
    union { float f; uint32_t u; } c;
    c.f = fmaf(x, 16384.0f, 12582912.0f + 16384.0f);
    return c.u & 0xFFF8u;
}
GEFEN_HD int lut_cell(float x) { return static_cast<int>(lut_byte_offset(x) >> 3); }

// Step 1, per threshold: its cell. -1 for thresholds below -1 (always exceeded), kLutCells + 1 for
// thresholds that x <= 1 can never exceed (also the +inf padding).
GEFEN_HD int lut_threshold_cell(float t) {
    if (t < -1.0f) return -1;
    if (!(t < 1.0f)) return kLutCells + 1;
    return lut_cell(t);
}
// Step 2, per cell: tcell[] is non-decreasing (thresholds are sorted), so two binary searches give
// the number of thresholds below the cell and inside it.
GEFEN_HD void lut_build_cell(int cell, const int* tcell, const float* thr, int nthr, float cb_last,
                             uint32_t* word_threshold, uint32_t* word_below) {
    int lo = 0, hi = nthr;
    while (lo < hi) { const int mid = (lo + hi) >> 1; if (tcell[mid] < cell) lo = mid + 1; else hi = mid; }
    const int below = lo;
    hi = nthr;
    while (lo < hi) { const int mid = (lo + hi) >> 1; if (tcell[mid] <= cell) lo = mid + 1; else hi = mid; }
    const int inside = lo - below;
    union { float f; uint32_t u; } c;
    c.f = inside >= 1 ? thr[below] : INFINITY;
    bool undecidable = inside >= 2;
    // cells that contain values above the last codebook entry need the non-monotone rule
    if (cb_last < 1.0f && (cb_last < -1.0f || cell >= lut_cell(cb_last))) undecidable = true;
    *word_threshold = c.u;
    *word_below = static_cast<uint32_t>(below) | (undecidable ? kLutSlowBit : 0u);
}

// The table query; *slow tells the caller to use entry_exact instead.
GEFEN_HD int lut_query(float x, const unsigned char* lut_bytes, bool* slow) {
    const uint2v e = *reinterpret_cast<const uint2v*>(lut_bytes + lut_byte_offset(x));
    union { float f; uint32_t u; } c;
    c.u = e.x;
    *slow = (e.y & kLutSlowBit) != 0u;
    return static_cast<int>(e.y & 0xFFu) + (x > c.f ? 1 : 0);
}

// Same, with the flag left in bit 31 of the result for the caller to test (several results can be
// OR-ed and tested once).
GEFEN_HD uint32_t lut_query_fast(float x, const unsigned char* lut_bytes) {
    const uint2v e = *reinterpret_cast<const uint2v*>(lut_bytes + lut_byte_offset(x));
    union { float f; uint32_t u; } c;
    c.u = e.x;
    return e.y + (x > c.f ? 1u : 0u);
}

// ---------------------------------------------------------------------------------------------
// a / b with b > 0 fixed per block and |a| <= b. `rb` must be the correctly rounded 1/b.
// q0 = a*rb is within one ulp; the exact remainder (one FMA) corrects it to the IEEE quotient.
// Valid while b, rb and the products stay normal; callers fall back to a true division outside
// [2^-100, 2^100] (see div_range_ok).
GEFEN_HD float div_by_block_constant(float a, float b, float rb) {
    const float q0 = a * rb;
    const float rem = fmaf(-q0, b, a);
    return fmaf(rem, rb, q0);
}
GEFEN_HD bool div_range_ok(float b) {
    return b >= 7.888609052210118e-31f && b <= 1.2676506002282294e+30f;
}

}  // namespace gefen
