// Shared first half of the weight-expansion passes: scatter the non-zeros of one work item into a shared-memory tile.
//
// A work item is (column chunk kc, R consecutive row-blocks).  Its dense tile lives in shared memory in the orientation
// of the destination (TR = false: lines are weight rows, cc columns long; TR = true: lines are weight columns, R * m rows
// long) and is all zeros when the item starts; the item's kept values are scattered into it straight from global memory
// (coalesced reads of val and idx).  What leaves the tile differs per pass: the dense expansion stores it as it is, the
// structured-sparse expansion compresses every aligned group of four reduction elements to two values plus metadata.
#pragma once
#include "nmg_common.cuh"

namespace nmg {

struct ExpandParams {
    const void *val;        // [tiles][C][g][n]
    const int16_t *idx;     // [tiles][C][g]
    const int8_t *order;    // [C][n]: row of slot t under pattern p
    void *dst;              // [planes][rows][ld] 16-bit
    int64_t ld, plane_elems;
    int64_t M, K, nb, nc;
    int n, m, g, C, cc;
    int R;                  // row-blocks per work item
    int pitch;              // elements per line of the shared-memory tile
};

constexpr int EXPAND_THREADS = 256;

// N_ = n for the vectorised scatter (1 or 2), 0 for the generic one.  `tile` is [lines][prm.pitch], `ord` the pattern
// table [C][n] in shared memory; rj = row-blocks of this item that exist (the last item of a chunk may hold fewer than R).
template <typename T, bool TR, int N_>
__device__ __forceinline__ void expand_scatter_item(const ExpandParams &prm, T *tile, const int8_t *ord, int64_t kc, int64_t mb0, int rj) {
    constexpr bool VEC_OK = N_ > 0;
    const int n = N_ > 0 ? N_ : prm.n, m = prm.m, g = prm.g, cc = prm.cc, pitch = prm.pitch;
    const T *val = static_cast<const T *>(prm.val);
    // tiles of consecutive row-blocks of one chunk are consecutive in memory
    const int64_t t0 = kc * prm.nb + mb0;
    const int16_t *isrc = prm.idx + t0 * cc;
    const T *vsrc = val + t0 * (int64_t)cc * n;
    auto scatter = [&](int e, int c, const T *v) {  // slot e of the item holds column c and the values v[0 .. n)
        if (c < 0 || c >= cc) return;  // a malformed index is ignored, never dereferenced
        const int j = e / cc, s = e - j * cc;
        const int8_t *o = ord + (s / g) * n;
        T *base = TR ? tile + c * pitch + j * m : tile + (j * m) * pitch + c;
        for (int t = 0; t < n; t++) base[TR ? o[t] : o[t] * pitch] = v[t];
    };
    const int total = rj * cc;
    bool vectorised = false;
    if constexpr (VEC_OK) if ((cc & 7) == 0) {
        vectorised = true;
        // eight slots per thread: one 16-byte load of indices and N_ 16-byte (16-bit) or 2 N_ (fp32) loads of values,
        // all issued before the first use, so a whole item's global loads are in flight together
        constexpr int VL = N_ * (int)sizeof(T) / 2;  // 16-byte loads of values per 8 slots
        const bool same_pattern = (g & 7) == 0;  // 8 consecutive slots then belong to one pattern
        for (int e8 = threadIdx.x * 8; e8 < total; e8 += EXPAND_THREADS * 8) {
            const uint4 iv = __ldg(reinterpret_cast<const uint4 *>(isrc + e8));
            uint4 vv[VL];
#pragma unroll
            for (int u = 0; u < VL; u++) vv[u] = __ldg(reinterpret_cast<const uint4 *>(vsrc + (int64_t)e8 * N_) + u);
            const int16_t *ci = reinterpret_cast<const int16_t *>(&iv);
            const T *vals = reinterpret_cast<const T *>(vv);
            const int j = e8 / cc, s0 = e8 - j * cc;  // cc is a multiple of 8: the 8 slots share the row-block
            if (same_pattern) {
                const int8_t *o = ord + (s0 / g) * N_;
                int off[N_];  // element offset of slot value t inside the tile, before the column is added
#pragma unroll
                for (int t = 0; t < N_; t++) off[t] = TR ? j * m + o[t] : (j * m + o[t]) * pitch;
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    const int c = ci[u];
                    if ((unsigned)c >= (unsigned)cc) continue;  // a malformed index is ignored, never dereferenced
#pragma unroll
                    for (int t = 0; t < N_; t++) tile[off[t] + (TR ? c * pitch : c)] = vals[u * N_ + t];
                }
            } else {
#pragma unroll
                for (int u = 0; u < 8; u++) scatter(e8 + u, ci[u], vals + u * N_);
            }
        }
    }
    if (!vectorised)
        for (int e = threadIdx.x; e < total; e += EXPAND_THREADS) scatter(e, isrc[e], vsrc + (int64_t)e * n);
}

}  // namespace nmg
