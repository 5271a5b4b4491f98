// Tensor-core matmul for fp16 / bf16 grouped n:m weights: tcgen05.mma with TMEM accumulators.
//
// In the format's orientation the n:m blocks run along the OUTPUT-feature axis of y = x W^T, so no operand of the
// forward product is structured-sparse along the reduction axis and tcgen05.mma.sp does not apply.  What the
// format does give is a weight that is 2/m .. n/m of its dense size in HBM and L2.  This kernel keeps it that
// way: the weight stays compressed in global memory (column-ordered copy: one pattern id + n values per
// (row-block, column)), is expanded tile by tile straight into the shared-memory operand layout of the
// tensor core (128-byte swizzle, K-major) by dedicated warps, and is multiplied at dense tensor-core rate
// against activation tiles that arrive by TMA.  The same kernel computes the transposed product dX = dY W: only
// the expansion routine differs (the tile is W^T, the reduction runs over weight rows).
//
// CTA = 14 warps: warp 0 issues TMA loads of the activation tile (256 tokens x 64 reduction elements), warp 1
// allocates TMEM and issues the MMAs (128 x 256 x 16, fp32 accumulate in TMEM), warps 2..13 form three groups
// that expand the weight tile (128 output features x 64 reduction elements) of every third k-block each; every
// group fetches its next tile's compressed data into registers before it scatters the current one.  Group 0 also runs the epilogue
// (tcgen05.ld -> bias -> convert -> store).  All waits are bounded; a wait that runs out sets the status word
// and the CTA drains to the common exit where TMEM is released.
#include <cstdlib>

#include "nmg_spmm_simt.cuh"
#include "nmg_tc_common.cuh"

namespace nmg {


struct TcParams {
    const uint16_t *pat;  // [nb][Kpn]
    const void *nval[3];  // [nb][Kpn][n] 16-bit values; fp32 weights: the hi / mid / lo bf16 planes
    const void *bias;     // [out_feats] or NULL
    void *out;
    int64_t out_feats;    // M (forward) or K (transposed)
    int64_t red;          // reduction length: K (forward) or M (transposed)
    int64_t ntok, ld_out, Kpn, nb;
    int out_token_major;  // 1: out[token][feature], 0: out[feature][token]
    int tiles_f, tiles_t; // output tiles along features / tokens
    int ksplit;           // > 1: the reduction axis is cut into ksplit ranges, one CTA each; fp32 partial tiles go to `partial`
    float *partial;       // [ksplit][tiles_f * 128][ld_partial] fp32, feature-major
    int64_t ld_partial;
    int *status;
};

// ---- weight-tile expansion ------------------------------------------------------------------------------
// A column of a row-block is n values plus a pattern id; its dense form (m halfs, n of them non-zero) is a byte
// permutation of the packed values and zero.  The per-pattern permutation selectors are tabulated once per CTA
// in shared memory: sel[p][q] is the PRMT selector that turns (v0 | v1 << 16, 0) into (row 2q | row 2q+1 << 16).
// Expansion is then M_/2 PRMTs per column, the tile is written with full-width, conflict-free stores, and no
// separate clearing pass exists.
//
// Swizzled K-major tile: element (row, e) lives at row*128 + (((e >> 3) ^ (row & 7)) << 4) + (e & 7)*2.
template <int M_> struct SelWords {  // the M_/2 16-bit selectors of one pattern, as 32-bit words
    static constexpr int W = M_ / 4;
    uint32_t w[W];
};
template <int M_> __device__ __forceinline__ SelWords<M_> load_sel(const uint16_t *sel, uint32_t p) {
    SelWords<M_> r;
    if constexpr (M_ == 4) r.w[0] = *reinterpret_cast<const uint32_t *>(sel + p * 2);
    else if constexpr (M_ == 8) { const uint2 v = *reinterpret_cast<const uint2 *>(sel + p * 4); r.w[0] = v.x; r.w[1] = v.y; }
    else { const uint4 v = *reinterpret_cast<const uint4 *>(sel + p * 8); r.w[0] = v.x; r.w[1] = v.y; r.w[2] = v.z; r.w[3] = v.w; }
    return r;
}
// rows (2q, 2q+1) of the column whose packed values are vv
template <int M_> __device__ __forceinline__ uint32_t expand_pair(const SelWords<M_> &s, uint32_t vv, int q) {
    return __byte_perm(vv, 0u, (q & 1) ? (s.w[q >> 1] >> 16) : (s.w[q >> 1] & 0xffffu));
}

// Forward: tile rows are weight rows feat0 .. feat0+127, tile columns are weight columns kb*64 .. +63.
// A thread owns one 8-column chunk (16 bytes of every tile row) of one row-block: lane = (row-block & 3) * 8 + chunk,
// warp w of the group takes row-blocks 4w .. 4w+3 (+16 per extra pass).  It loads the chunk's 8 pattern ids and
// 8*n values with 16-byte loads, expands them with PRMTs and writes every row of the row-block with one 16-byte
// store; the 8 lanes that share a row cover its 128 bytes, so stores are conflict-free.
template <int N_, int M_> struct FwdRegs {
    static constexpr int RB = TC_BM / M_;               // row-blocks per tile
    static constexpr int PASSES = (RB + 15) / 16;       // 16 row-blocks per pass of the group's 4 warps
    uint4 pat[PASSES];                                   // 8 pattern ids (16 bits each); .x = 0xffffffff marks "no row-block"
    uint4 val[PASSES][N_];                               // 8 * n halfs
};

template <int N_, int M_>
__device__ __forceinline__ void fetch_forward(FwdRegs<N_, M_> &t, const TcParams &prm, const void *plane, int64_t feat0, int64_t kb,
                                              int gwarp, int lane) {
    constexpr int RB = FwdRegs<N_, M_>::RB;
    const uint16_t *nval = static_cast<const uint16_t *>(plane);
    const int c8 = lane & 7;
#pragma unroll
    for (int i = 0; i < FwdRegs<N_, M_>::PASSES; i++) {
        const int rbl = i * 16 + gwarp * 4 + (lane >> 3);
        const int64_t mb = feat0 / M_ + rbl;
        if (rbl < RB && mb < prm.nb) {
            const int64_t e0 = mb * prm.Kpn + kb * TC_BK + c8 * 8;
            t.pat[i] = __ldg(reinterpret_cast<const uint4 *>(prm.pat + e0));
#pragma unroll
            for (int q = 0; q < N_; q++) t.val[i][q] = __ldg(reinterpret_cast<const uint4 *>(nval + e0 * N_) + q);
        } else {
            t.pat[i] = make_uint4(0xffffffffu, 0, 0, 0);
#pragma unroll
            for (int q = 0; q < N_; q++) t.val[i][q] = make_uint4(0, 0, 0, 0);
        }
    }
}

template <int N_, int M_>
__device__ __forceinline__ void write_forward(const FwdRegs<N_, M_> &t, char *a_tile, const uint16_t *sel, int gwarp, int lane) {
    constexpr int C = (int)comb(N_, M_);
    constexpr int RB = FwdRegs<N_, M_>::RB;
    const int c8 = lane & 7;
#pragma unroll
    for (int i = 0; i < FwdRegs<N_, M_>::PASSES; i++) {
        const int rbl = i * 16 + gwarp * 4 + (lane >> 3);
        if (rbl >= RB) continue;
        const int row0 = rbl * M_;
        const bool live = t.pat[i].x != 0xffffffffu;
        const uint32_t pw[4] = {t.pat[i].x, t.pat[i].y, t.pat[i].z, t.pat[i].w};
        uint32_t pid[8];  // clamped pattern ids of the 8 columns
        uint32_t v[8];    // packed values (slot 0 | slot 1 << 16) of the 8 columns
#pragma unroll
        for (int c = 0; c < 8; c++) pid[c] = min(live ? ((pw[c >> 1] >> ((c & 1) * 16)) & 0xffffu) : 0u, (uint32_t)(C - 1));
        if (N_ == 2) {
            const uint32_t a[8] = {t.val[i][0].x, t.val[i][0].y, t.val[i][0].z, t.val[i][0].w,
                                   t.val[i][N_ - 1].x, t.val[i][N_ - 1].y, t.val[i][N_ - 1].z, t.val[i][N_ - 1].w};
#pragma unroll
            for (int c = 0; c < 8; c++) v[c] = a[c];
        } else {
            const uint32_t a[4] = {t.val[i][0].x, t.val[i][0].y, t.val[i][0].z, t.val[i][0].w};
#pragma unroll
            for (int c = 0; c < 8; c++) v[c] = (a[c >> 1] >> ((c & 1) * 16)) & 0xffffu;
        }
        char *rowp = a_tile + row0 * 128;
        const uint32_t cx = (uint32_t)((c8 ^ (row0 & 7)) << 4);  // chunk offset of row row0; row r adds (r - row0) under the xor
#pragma unroll
        for (int w = 0; w < M_ / 4; w++) {  // one selector word (rows 4w .. 4w+3) at a time keeps the live registers few
            uint32_t sw[8];
#pragma unroll
            for (int c = 0; c < 8; c++) sw[c] = *reinterpret_cast<const uint32_t *>(sel + pid[c] * (M_ / 2) + 2 * w);
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const int q = 2 * w + h;
                uint32_t e[8];  // rows (2q | 2q+1 << 16) of each column
#pragma unroll
                for (int c = 0; c < 8; c++) e[c] = live ? __byte_perm(v[c], 0u, h ? (sw[c] >> 16) : sw[c]) : 0u;
                const uint4 lo = make_uint4(__byte_perm(e[0], e[1], 0x5410), __byte_perm(e[2], e[3], 0x5410),
                                            __byte_perm(e[4], e[5], 0x5410), __byte_perm(e[6], e[7], 0x5410));
                const uint4 hi = make_uint4(__byte_perm(e[0], e[1], 0x7632), __byte_perm(e[2], e[3], 0x7632),
                                            __byte_perm(e[4], e[5], 0x7632), __byte_perm(e[6], e[7], 0x7632));
                // row0 is a multiple of 4, so (row0 + k) & 7 == (row0 & 7) ^ k for k < 4, and for M_ >= 8 row0 & 7 == 0
                *reinterpret_cast<uint4 *>(rowp + (2 * q) * 128 + (cx ^ (uint32_t)(((2 * q) & 7) << 4))) = lo;
                *reinterpret_cast<uint4 *>(rowp + (2 * q + 1) * 128 + (cx ^ (uint32_t)(((2 * q + 1) & 7) << 4))) = hi;
            }
        }
    }
}

// Transposed: tile rows are weight columns feat0 .. feat0+127 (one per thread of the group), the tile's K axis is
// weight rows kb*64 .. +63, i.e. 64/m row-blocks whose expanded columns lie side by side in the thread's row.
template <int N_, int M_> struct TrRegs {
    static constexpr int E = TC_BK / M_;  // row-blocks per k-block
    uint32_t pat[E];                       // 0xffffffff = row-block past the end of the weight
    uint32_t val[E];                       // n <= 2 halfs
};

template <int N_, int M_>
__device__ __forceinline__ void fetch_transposed(TrRegs<N_, M_> &t, const TcParams &prm, const void *plane, int64_t feat0, int64_t kb,
                                                 int row) {
    constexpr int E = TrRegs<N_, M_>::E;
    const int64_t kg = feat0 + row;
    const uint16_t *nval = static_cast<const uint16_t *>(plane);
#pragma unroll
    for (int j = 0; j < E; j++) {
        const int64_t mb = kb * E + j;
        t.pat[j] = 0xffffffffu;
        t.val[j] = 0;
        if (mb < prm.nb) {
            const int64_t e = mb * prm.Kpn + kg;
            t.pat[j] = __ldg(prm.pat + e);
            if (N_ == 2) t.val[j] = __ldg(reinterpret_cast<const uint32_t *>(nval + e * 2));
            else t.val[j] = __ldg(nval + e);
        }
    }
}

template <int N_, int M_>
__device__ __forceinline__ void write_transposed(const TrRegs<N_, M_> &t, char *a_tile, const uint16_t *sel, int row) {
    constexpr int C = (int)comb(N_, M_);
    constexpr int E = TrRegs<N_, M_>::E;
    constexpr int WPE = M_ / 2;  // 32-bit words per expanded column
    uint32_t w[TC_BK / 2];       // the thread's whole tile row
#pragma unroll
    for (int j = 0; j < E; j++) {
        const bool live = t.pat[j] != 0xffffffffu;
        const SelWords<M_> s = load_sel<M_>(sel, min(t.pat[j], (uint32_t)(C - 1)));
#pragma unroll
        for (int q = 0; q < WPE; q++) w[j * WPE + q] = live ? expand_pair<M_>(s, t.val[j], q) : 0u;
    }
    char *rowp = a_tile + row * 128;
#pragma unroll
    for (int c = 0; c < 8; c++)
        *reinterpret_cast<uint4 *>(rowp + (((c ^ row) & 7) << 4)) = make_uint4(w[4 * c], w[4 * c + 1], w[4 * c + 2], w[4 * c + 3]);
}


// ---- the kernel -------------------------------------------------------------------------------------------
template <int N_, int M_, typename T, bool TRANSPOSED>
__global__ void __launch_bounds__(TC_THREADS, 1)
spmm_tc_kernel(const TcParams prm, const __grid_constant__ CUtensorMap tmap0, const __grid_constant__ CUtensorMap tmap1,
               const __grid_constant__ CUtensorMap tmap2) {
    constexpr int TERMS = TcMode<T>::TERMS;
    using E = typename TcMode<T>::elem;  // element type the tensor cores see
    static_assert((3 * TC_STAGES + 2) * 8 <= 120, "barriers overlap the TMEM slot");
    static_assert(TC_BM % (4 * M_) == 0 && TC_BK % M_ == 0 && M_ % 4 == 0 && N_ <= 2, "tile must hold whole row-blocks; pattern rows are packed in 32 bits");
    constexpr Order<N_, M_> ORD{};
    constexpr int C = Order<N_, M_>::C;

    constexpr bool SPLIT = TERMS > 1;
    constexpr int GROUPS = TcMode<T>::GROUPS;
    constexpr uint32_t TMEM_COLS = SPLIT ? 2 * TC_ACC_COLS : TC_ACC_COLS;

    extern __shared__ char smem_raw[];
    char *smem = reinterpret_cast<char *>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    char *a_stages = smem;
    char *b_stages = smem + TC_STAGES * TC_A_BYTES;
    char *misc = smem + TC_STAGES * (TC_A_BYTES + TC_B_BYTES);  // 1024-byte aligned: barriers first
    uint64_t *full_a = reinterpret_cast<uint64_t *>(misc);
    uint64_t *full_b = full_a + TC_STAGES;
    uint64_t *empty = full_b + TC_STAGES;
    uint64_t *chunk_done = empty + TC_STAGES;  // MMA -> promotion / epilogue: the accumulator tile is complete
    uint64_t *promoted = chunk_done + 1;       // promotion -> MMA: the accumulator tile may be overwritten
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(misc + 120);
    uint16_t *sel = reinterpret_cast<uint16_t *>(misc + 128);  // [C][M_/2] PRMT selectors, 16-byte aligned

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // Few output tiles (few tokens): the grid is ksplit x tiles and every CTA takes one range of the reduction axis, so
    // that the compressed weight streams from HBM through all SMs; a second kernel adds the partial tiles.
    const int ntiles = prm.tiles_f * prm.tiles_t;
    const int split = (int)blockIdx.x / ntiles;
    int tile_f, tile_t;
    tile_of_cta((int)blockIdx.x - split * ntiles, prm.tiles_f, prm.tiles_t, tile_f, tile_t);
    const int64_t tok0 = (int64_t)tile_t * TC_BN;
    const int64_t feat0 = (int64_t)tile_f * TC_BM;
    // 32-bit loop arithmetic throughout: the single MMA-issuing thread must stay ahead of the tensor core, and a
    // 64-bit division per iteration on that thread is enough to make issue the bottleneck.
    const int nkb_all = (int)((prm.red + TC_BK - 1) / TC_BK) * TERMS;  // iterations: k-blocks x split terms (term fastest)
    const int kb_per = (nkb_all + prm.ksplit - 1) / prm.ksplit;
    const int kb_base = split * kb_per;                                 // this CTA's first iteration (0 unless ksplit > 1)
    const int nkb = (nkb_all < kb_base + kb_per ? nkb_all : kb_base + kb_per) - kb_base;  // >= 1 by the host's choice of ksplit
    const int chunk_it = SPLIT ? TC_CHUNK_KB * TERMS : nkb;          // iterations per accumulation chunk
    const int nchunks = (nkb + chunk_it - 1) / chunk_it;

    if (tid == 0) {
        for (int s = 0; s < TC_STAGES; s++) {
            mbar_init(&full_a[s], 128);
            mbar_init(&full_b[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(chunk_done, 1);
        mbar_init(promoted, 128);
        mbar_fence_init();
    }
    for (int e = tid; e < C * (M_ / 2); e += TC_THREADS) {
        // selector for rows (2q, 2q+1) of pattern p: bytes of slot 0 are 0,1, of slot 1 are 2,3, byte 4 is zero
        const int p = e / (M_ / 2), q = e - p * (M_ / 2);
        uint32_t code = 0;
        for (int h = 0; h < 2; h++) {
            uint32_t nib = 0x44;
            for (int sl = 0; sl < N_; sl++)
                if (ORD.v[p * Order<N_, M_>::LD + sl] == 2 * q + h) nib = sl == 0 ? 0x10 : 0x32;
            code |= nib << (8 * h);
        }
        sel[e] = (uint16_t)code;
    }
    if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // Promotion + epilogue, run by four warps that together cover the 128 TMEM lanes.  For every finished chunk the
    // accumulator tile is added to the running tile (columns 256..511) with round-to-nearest adds; the last chunk is
    // added, biased, converted and stored to global memory instead.  16-bit mode has a single chunk.
    // Bias, convert and store one 32-column slice (32 tokens) of this thread's feature row.
    auto store_slice = [&](const uint32_t (&r)[32], int sl, int64_t feat, float b) {
        T *out = static_cast<T *>(prm.out);
        const int64_t tokc = tok0 + sl * 32;
        const bool vec = !prm.out_token_major && tokc + 32 <= prm.ntok && (prm.ld_out % (16 / (int)sizeof(T))) == 0 &&
                         (reinterpret_cast<uintptr_t>(out) & 15) == 0;
        if (vec) {  // 32 consecutive tokens of this feature: 16-byte stores
            uint4 *dst = reinterpret_cast<uint4 *>(out + feat * prm.ld_out + tokc);
            if constexpr (sizeof(T) == 4) {
#pragma unroll
                for (int v = 0; v < 8; v++)
                    dst[v] = make_uint4(__float_as_uint(__uint_as_float(r[4 * v]) + b), __float_as_uint(__uint_as_float(r[4 * v + 1]) + b),
                                        __float_as_uint(__uint_as_float(r[4 * v + 2]) + b), __float_as_uint(__uint_as_float(r[4 * v + 3]) + b));
            } else {
#pragma unroll
                for (int v = 0; v < 4; v++) {
                    uint32_t w[4];
#pragma unroll
                    for (int h = 0; h < 4; h++) {
                        const T lo = DT<T>::from_f32(__uint_as_float(r[8 * v + 2 * h]) + b);
                        const T hi = DT<T>::from_f32(__uint_as_float(r[8 * v + 2 * h + 1]) + b);
                        w[h] = (uint32_t)bits16<T>(lo) | ((uint32_t)bits16<T>(hi) << 16);
                    }
                    dst[v] = make_uint4(w[0], w[1], w[2], w[3]);
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; j++) {
                const int64_t tok = tokc + j;
                if (tok < prm.ntok) {
                    const T o = DT<T>::from_f32(__uint_as_float(r[j]) + b);
                    if (prm.out_token_major) out[tok * prm.ld_out + feat] = o;
                    else out[feat * prm.ld_out + tok] = o;
                }
            }
        }
    };

    // 16-bit mode: one accumulation chunk, so the four draining warps only run the epilogue.
    auto epilogue_once = [&]() {
        if (!mbar_wait_bounded(chunk_done, 0, prm.status, 15)) return;
        tc_fence_after();
        const int q = warp & 3;  // TMEM lane quarter this warp may read
        const int64_t feat = feat0 + q * 32 + lane;
        const bool feat_ok = feat < prm.out_feats;
        const float b = (prm.bias && feat_ok) ? DT<T>::to_f32(static_cast<const T *>(prm.bias)[feat]) : 0.f;
        for (int sl = 0; sl < TC_BN / 32; sl++) {
            uint32_t r[32];
            tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(sl * 32), r);
            if (tok0 + sl * 32 >= prm.ntok) continue;  // warp-uniform
            if (prm.ksplit > 1) {  // raw fp32 partial sums; rows exist for every feature of the tile, ld_partial covers the slice
                uint4 *dst = reinterpret_cast<uint4 *>(prm.partial + ((int64_t)split * prm.tiles_f * TC_BM + feat) * prm.ld_partial + tok0 + sl * 32);
#pragma unroll
                for (int v = 0; v < 8; v++) dst[v] = make_uint4(r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]);
                continue;
            }
            if (feat_ok) store_slice(r, sl, feat, b);
        }
        tc_fence_before();
    };

    // fp32 mode: for every finished chunk the accumulator tile is added to the running tile (columns 256..511) with
    // round-to-nearest adds; the last chunk is added and stored to global memory instead.
    auto drain_chunk = [&](int c) -> bool {
        const int q = warp & 3;
        const int64_t feat = feat0 + q * 32 + lane;
        const bool feat_ok = feat < prm.out_feats;
        const float b = (prm.bias && feat_ok) ? DT<T>::to_f32(static_cast<const T *>(prm.bias)[feat]) : 0.f;
        const uint32_t lane_base = tmem_base + ((uint32_t)(q * 32) << 16);
        if (!mbar_wait_bounded(chunk_done, (uint32_t)(c & 1), prm.status, 15)) return false;
        tc_fence_after();
        const bool last = c == nchunks - 1;
        for (int sl = 0; sl < TC_BN / 32; sl++) {
            uint32_t r[32];
            tmem_ld32(lane_base + (uint32_t)(sl * 32), r);
            if (c > 0) {
                uint32_t run[32];
                tmem_ld32(lane_base + (uint32_t)(TC_ACC_COLS + sl * 32), run);
#pragma unroll
                for (int j = 0; j < 32; j++) r[j] = __float_as_uint(__fadd_rn(__uint_as_float(run[j]), __uint_as_float(r[j])));
            }
            if (!last) {
                tmem_st32(lane_base + (uint32_t)(TC_ACC_COLS + sl * 32), r);
                continue;
            }
            if (tok0 + sl * 32 < prm.ntok && feat_ok) store_slice(r, sl, feat, b);
        }
        tc_fence_before();
        if (!last) mbar_arrive(promoted);
        return true;
    };

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (one lane)
        if (lane == 0) {
            for (int kb = 0; kb < nkb; kb++) {
                const int s = kb % TC_STAGES;
                const uint32_t ph = (uint32_t)((kb / TC_STAGES) & 1);
                if (!mbar_wait_bounded(&empty[s], ph ^ 1, prm.status, 11)) break;
                mbar_expect_tx(&full_b[s], TC_B_BYTES);
                const int xc = TERMS == 1 ? 0 : kSplitX[kb % TERMS];
                const CUtensorMap *tm = xc == 0 ? &tmap0 : (xc == 1 ? &tmap1 : &tmap2);
                tma_load_2d(b_stages + s * TC_B_BYTES, tm, ((kb_base + kb) / TERMS) * TC_BK, (int)tok0, &full_b[s]);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (one lane)
        if (lane == 0) {
            const uint32_t idesc = make_idesc<E>();
            bool ok = true;
            int chunk = 0, in_chunk = 0;  // position inside the accumulation chunk, kept without divisions
            for (int kb = 0; kb < nkb && ok; kb++) {
                const int s = kb % TC_STAGES;
                const uint32_t ph = (uint32_t)((kb / TC_STAGES) & 1);
                const bool first = in_chunk == 0;
                if (first && chunk > 0) ok = mbar_wait_bounded(promoted, (uint32_t)((chunk - 1) & 1), prm.status, 16);
                ok = ok && mbar_wait_bounded(&full_a[s], ph, prm.status, 12) && mbar_wait_bounded(&full_b[s], ph, prm.status, 13);
                if (!ok) break;
                tc_fence_after();
                const uint64_t adesc = make_sw128_desc(smem_u32(a_stages + s * TC_A_BYTES));
                const uint64_t bdesc = make_sw128_desc(smem_u32(b_stages + s * TC_B_BYTES));
#pragma unroll
                for (int k = 0; k < TC_BK / 16; k++)  // 16 elements = 32 bytes = 2 descriptor units per step
                    tc_mma_f16(tmem_base, adesc + 2 * k, bdesc + 2 * k, idesc, (first && k == 0) ? 0u : 1u);
                tc_commit(&empty[s]);  // arrives when the MMAs above have read the stage
                if (++in_chunk == chunk_it || kb + 1 == nkb) {
                    tc_commit(chunk_done);
                    in_chunk = 0;
                    chunk++;
                }
            }
            if (!ok) tc_commit(chunk_done);  // error path: let the drain warps fall through their bounded wait sooner
        }
    } else {
        // ------------------------------------------------------------------ expansion groups
        const int group = (warp - 2) >> 2;
        const int gwarp = (warp - 2) & 3;
        const int gtid = tid - 64 - group * 128;
        // Two register buffers in ping-pong: the global loads of the group's next tile are in flight while the
        // current one is written, and nothing is copied between the buffers.
        int drained = 0;  // group 0: accumulation chunks already promoted
        auto run_group = [&](auto fetch, auto write, auto &buf_a, auto &buf_b) {
            auto publish = [&](int kb, auto &buf) -> bool {
                const int s = kb % TC_STAGES;
                const uint32_t ph = (uint32_t)((kb / TC_STAGES) & 1);
                if (SPLIT && group == 0) {
                    // Before feeding a later chunk, promote the finished ones: the MMAs of a chunk depend only on
                    // tiles that are already published, so this wait cannot deadlock, and the MMA issuer needs
                    // the promotion before it may restart the accumulator.
                    while (drained < kb / chunk_it) {
                        if (!drain_chunk(drained)) return false;
                        drained++;
                    }
                }
                if (!mbar_wait_bounded(&empty[s], ph ^ 1, prm.status, 14)) return false;
                write(buf, a_stages + s * TC_A_BYTES);
                fence_proxy_async_smem();  // generic-proxy stores -> visible to the tensor core's async-proxy reads
                mbar_arrive(&full_a[s]);
                return true;
            };
            if (group < nkb) fetch(buf_a, group);
            for (int kb = group; kb < nkb; kb += 2 * GROUPS) {
                if (kb + GROUPS < nkb) fetch(buf_b, kb + GROUPS);
                if (!publish(kb, buf_a)) break;
                if (kb + GROUPS >= nkb) break;
                if (kb + 2 * GROUPS < nkb) fetch(buf_a, kb + 2 * GROUPS);
                if (!publish(kb + GROUPS, buf_b)) break;
            }
        };
        if (TRANSPOSED) {
            TrRegs<N_, M_> ra, rb;
            run_group([&](TrRegs<N_, M_> &t, int it) {
                          fetch_transposed<N_, M_>(t, prm, prm.nval[TERMS == 1 ? 0 : kSplitW[it % TERMS]], feat0, (kb_base + it) / TERMS, gtid);
                      },
                      [&](const TrRegs<N_, M_> &t, char *tile) { write_transposed<N_, M_>(t, tile, sel, gtid); }, ra, rb);
        } else {
            FwdRegs<N_, M_> ra, rb;
            run_group([&](FwdRegs<N_, M_> &t, int it) {
                          fetch_forward<N_, M_>(t, prm, prm.nval[TERMS == 1 ? 0 : kSplitW[it % TERMS]], feat0, (kb_base + it) / TERMS, gwarp, lane);
                      },
                      [&](const FwdRegs<N_, M_> &t, char *tile) { write_forward<N_, M_>(t, tile, sel, gwarp, lane); }, ra, rb);
        }
        if (group == 0) {
            if constexpr (SPLIT) {
                while (drained < nchunks && drain_chunk(drained)) drained++;  // remaining promotions, then the result
            } else {
                epilogue_once();
            }
        }
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ------------------------------------------------------------------------------------------------------ host side
bool tc_supported(const Geo &geo, int dtype) {
    if (dtype != NMG_F16 && dtype != NMG_BF16 && dtype != NMG_F32) return false;
    return (geo.n == 1 && geo.m == 4) || (geo.n == 2 && geo.m == 4) || (geo.n == 1 && geo.m == 8) || (geo.n == 2 && geo.m == 8) ||
           (geo.n == 1 && geo.m == 16);
}

static size_t tc_smem_bytes(int C) {
    return (size_t)TC_STAGES * (TC_A_BYTES + TC_B_BYTES) + 128 + (size_t)C * 16 + 1024;
}

// ---- fp32 activations: three bf16 planes [3][rows][ldp], written by one elementwise pass ---------------------------
__global__ void __launch_bounds__(128) split_f32_kernel(const float *__restrict__ src, int64_t rows, int64_t cols, int64_t ld_src,
                                                        __nv_bfloat16 *__restrict__ dst, int64_t ldp, int64_t plane_elems) {
    const int64_t r = blockIdx.y;
    const float *row = src + r * ld_src;
    const bool vec = (reinterpret_cast<uintptr_t>(row) & 15) == 0;
    // eight elements per thread: two 16-byte loads, one 16-byte store per plane (ldp is a multiple of 8)
    for (int64_t c = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 8; c < ldp; c += (int64_t)gridDim.x * blockDim.x * 8) {
        float f[8];
        if (vec && c + 8 <= cols) {
            const float4 a = __ldg(reinterpret_cast<const float4 *>(row + c)), b = __ldg(reinterpret_cast<const float4 *>(row + c + 4));
            f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
        } else {
#pragma unroll
            for (int i = 0; i < 8; i++) f[i] = c + i < cols ? row[c + i] : 0.f;
        }
        uint32_t w[3][4];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const __nv_bfloat16 hi = __float2bfloat16_rn(f[i]);
            const float r1 = f[i] - __bfloat162float(hi);
            const __nv_bfloat16 mid = __float2bfloat16_rn(r1);
            const __nv_bfloat16 lo = __float2bfloat16_rn(r1 - __bfloat162float(mid));
            const uint32_t sh = (i & 1) * 16;
            if (!(i & 1)) { w[0][i >> 1] = 0; w[1][i >> 1] = 0; w[2][i >> 1] = 0; }
            w[0][i >> 1] |= (uint32_t)__bfloat16_as_ushort(hi) << sh;
            w[1][i >> 1] |= (uint32_t)__bfloat16_as_ushort(mid) << sh;
            w[2][i >> 1] |= (uint32_t)__bfloat16_as_ushort(lo) << sh;
        }
        const int64_t o = r * ldp + c;
#pragma unroll
        for (int p = 0; p < 3; p++) *reinterpret_cast<uint4 *>(dst + p * plane_elems + o) = make_uint4(w[p][0], w[p][1], w[p][2], w[p][3]);
    }
}

// ---- split-K of the fused kernel for few output tiles ----------------------------------------------------------------
// Policy (pure arithmetic, so that workspace queries need no device): with fewer output tiles than half the SMs of a
// B200 the reduction axis is cut so that about one CTA per SM runs, every range keeping at least four k-blocks.
constexpr int TC_POLICY_SMS = 148;
int tc_ksplit(const Geo &geo, int dtype, bool transposed, int64_t tokens) {
    if (dtype == NMG_F32) return 1;  // fp32 mode accumulates in promoted chunks inside one CTA
    const int64_t feats = transposed ? geo.K : geo.M, red = transposed ? geo.M : geo.K;
    const int64_t tiles = ((feats + TC_BM - 1) / TC_BM) * ((tokens + TC_BN - 1) / TC_BN);
    const int64_t nkb = (red + TC_BK - 1) / TC_BK;
    if (tiles * 2 > TC_POLICY_SMS || nkb < 8) return 1;
    int64_t want = TC_POLICY_SMS / tiles;
    if (want > nkb / 4) want = nkb / 4;
    if (want > 32) want = 32;
    if (want < 2) return 1;
    const int64_t per = (nkb + want - 1) / want;
    return (int)((nkb + per - 1) / per);  // every range non-empty
}
size_t tc_ksplit_workspace_bytes(const Geo &geo, int dtype, bool transposed, int64_t tokens) {
    const int ks = tc_ksplit(geo, dtype, transposed, tokens);
    if (ks <= 1) return 0;
    const int64_t feats = transposed ? geo.K : geo.M;
    return (size_t)ks * (size_t)round_up(feats, TC_BM) * (size_t)round_up(tokens, TC_BN) * 4 + 512;
}

// out = sum over the ranges of partial[s] (+ bias), converted; 32 x 32 tiles through shared memory so that both the reads
// (tokens contiguous) and token-major writes (features contiguous) are coalesced.  Ranges are added in a fixed order.
template <typename T>
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float *__restrict__ partial, int ksplit, int64_t plane, int64_t ldp,
                                                            int64_t feats, int64_t ntok, const T *__restrict__ bias, T *__restrict__ out,
                                                            int64_t ld_out, int token_major) {
    __shared__ float tile[32][33];
    const int64_t f0 = (int64_t)blockIdx.y * 32, t0 = (int64_t)blockIdx.x * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    for (int r = ty; r < 32; r += 8) {
        const int64_t f = f0 + r, t = t0 + tx;
        float acc = 0.f;
        if (f < feats && t < ntok) {
            for (int s = 0; s < ksplit; s++) acc += partial[s * plane + f * ldp + t];
            if (bias) acc += DT<T>::to_f32(bias[f]);
        }
        tile[r][tx] = acc;
    }
    __syncthreads();
    if (token_major) {
        for (int r = ty; r < 32; r += 8) {  // r = token, tx = feature
            const int64_t t = t0 + r, f = f0 + tx;
            if (f < feats && t < ntok) out[t * ld_out + f] = DT<T>::from_f32(tile[tx][r]);
        }
    } else {
        for (int r = ty; r < 32; r += 8) {
            const int64_t f = f0 + r, t = t0 + tx;
            if (f < feats && t < ntok) out[f * ld_out + t] = DT<T>::from_f32(tile[r][tx]);
        }
    }
}

size_t tc_split_workspace_bytes(const Geo &geo, int dtype, bool transposed, int64_t tokens) {
    if (dtype != NMG_F32) return 0;
    const int64_t red = transposed ? geo.M : geo.K;
    return (size_t)3 * (size_t)tokens * (size_t)round_up(red, 8) * 2 + 512;
}

template <int N_, int M_, typename T, bool TR>
static int tc_launch_one(const TcParams &p, const CUtensorMap *tm, cudaStream_t st) {
    const size_t smem = tc_smem_bytes((int)comb(N_, M_));
    const int64_t ctas = (int64_t)p.tiles_f * p.tiles_t * p.ksplit;
    if (ctas > 0x7fffffff) NMG_FAIL(NMG_ERR_UNSUPPORTED, "too many output tiles for one launch");
    dim3 grid((unsigned)ctas);
    NMG_CUDA(cudaFuncSetAttribute(spmm_tc_kernel<N_, M_, T, TR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    spmm_tc_kernel<N_, M_, T, TR><<<grid, TC_THREADS, smem, st>>>(p, tm[0], tm[1], tm[2]);
    NMG_CUDA(cudaGetLastError());
    return NMG_OK;
}

template <int N_, int M_>
static int tc_launch_nm(int dtype, bool transposed, const TcParams &p, const CUtensorMap *tm, cudaStream_t st) {
    if (dtype == NMG_F16) return transposed ? tc_launch_one<N_, M_, __half, true>(p, tm, st) : tc_launch_one<N_, M_, __half, false>(p, tm, st);
    if (dtype == NMG_F32) return transposed ? tc_launch_one<N_, M_, float, true>(p, tm, st) : tc_launch_one<N_, M_, float, false>(p, tm, st);
    return transposed ? tc_launch_one<N_, M_, __nv_bfloat16, true>(p, tm, st) : tc_launch_one<N_, M_, __nv_bfloat16, false>(p, tm, st);
}

// Policy of the two tensor-core variants.
bool tc_use_dense(const Geo &geo, int dtype, int64_t tokens) {
    const bool fused = tc_supported(geo, dtype), dense = tc_dense_supported(geo, dtype);
    if (!dense) return false;
    if (!fused) return true;
    // Measured crossover (4096^2 and 16384^2 bf16 weights): a tie around 1024 tokens (0.055 / 0.053 ms and 0.567 / 0.598 ms,
    // fused / two-pass), two passes clearly ahead at 1536 (0.099 / 0.072 ms and 0.836 / 0.799 ms); fp32 (six split products,
    // so six in-kernel expansions per tile) prefers two passes from 256 tokens.
    return tokens >= (dtype == NMG_F32 ? 256 : 1280);
}

// act: [tokens][ld_act] with the reduction axis contiguous (X for the forward, dY for the transposed product).
int tc_matmul(const Geo &geo, int dtype, bool transposed, bool dense, const void *val, const int16_t *idx, const uint16_t *pat,
              const void *nval, const void *act, int64_t ld_act, int64_t tokens, const void *bias, void *const *outs, int n_outs,
              void *mc_out, int64_t ld_out, int out_token_major, void *ws, size_t ws_bytes, cudaStream_t st, const Epilogue &epi) {
    if (n_outs < 1 || (n_outs > 1 && !dense)) NMG_FAIL(NMG_ERR_UNSUPPORTED, "several output buffers need the two-pass tensor-core variant");
    void *out = outs[0];
    const int64_t red = transposed ? geo.M : geo.K;
    // the two-pass variant on CTA pairs loads the activation tile in two halves of 128 tokens
    const uint32_t box_tok = (dense && tc_dense_uses_pair(geo, dtype, transposed)) ? 128 : TC_BN;
    CUtensorMap tm[3];
    int rc;
    const void *planes[3] = {nval, nval, nval};
    if (dtype == NMG_F32) {
        const size_t need = tc_split_workspace_bytes(geo, dtype, transposed, tokens);
        if (!ws || ws_bytes < need) NMG_FAIL(NMG_ERR_WORKSPACE, "workspace of %zu bytes required for the split activation, got %zu", need, ws_bytes);
        __nv_bfloat16 *xs = reinterpret_cast<__nv_bfloat16 *>(((uintptr_t)ws + 255) & ~(uintptr_t)255);
        const int64_t ldp = round_up(red, 8);
        const int64_t plane_elems = tokens * ldp;
        if (tokens > 65535 * 16) NMG_FAIL(NMG_ERR_UNSUPPORTED, "too many tokens for the split pre-pass");
        for (int64_t r0 = 0; r0 < tokens; r0 += 65535) {  // grid.y limit
            const int64_t nr = tokens - r0 < 65535 ? tokens - r0 : 65535;
            const int64_t bx = (ldp / 8 + 127) / 128;
            dim3 grid((unsigned)(bx > 64 ? 64 : bx), (unsigned)nr);
            split_f32_kernel<<<grid, 128, 0, st>>>(static_cast<const float *>(act) + r0 * ld_act, nr, red, ld_act, xs + r0 * ldp, ldp, plane_elems);
        }
        NMG_CUDA(cudaGetLastError());
        for (int c = 0; c < 3; c++)
            if ((rc = encode_tmap_2d(&tm[c], NMG_BF16, xs + c * plane_elems, (uint64_t)red, (uint64_t)tokens, (uint64_t)ldp, TC_BK, box_tok, 1))) return rc;
        if (!dense) {
            const NaturalLayout lay = natural_layout(geo, dtype);
            for (int c = 0; c < 3; c++) planes[c] = static_cast<const char *>(nval) + lay.val_bytes + c * lay.plane_bytes;
        }
        ws = static_cast<char *>(ws) + need;  // what follows the split activation is free for the expanded weight
        ws_bytes -= need;
    } else {
        if ((rc = encode_tmap_2d(&tm[0], dtype, act, (uint64_t)red, (uint64_t)tokens, (uint64_t)ld_act, TC_BK, box_tok, 1))) return rc;
        tm[1] = tm[0];
        tm[2] = tm[0];
    }
    if (dense) {
        const ProfileEvents pe = take_profile_events();
        if (pe.start) NMG_CUDA(cudaEventRecord(pe.start, st));
        rc = tc_dense_matmul(geo, dtype, transposed, val, idx, tm, tokens, bias, outs, n_outs, mc_out, ld_out, out_token_major, ws, ws_bytes, st, epi);
        if (rc == NMG_OK && pe.stop) NMG_CUDA(cudaEventRecord(pe.stop, st));
        return rc;
    }
    int *status = nullptr;
    if ((rc = get_status_word(&status))) return rc;
    const int64_t feats = transposed ? geo.K : geo.M;
    const int64_t ftile = TC_BM;
    TcParams p{};
    p.pat = pat;
    for (int c = 0; c < 3; c++) p.nval[c] = planes[c];
    p.bias = bias; p.out = out; p.out_feats = feats; p.red = red; p.ntok = tokens; p.ld_out = ld_out;
    p.Kpn = natural_width(geo); p.nb = geo.nb; p.out_token_major = out_token_major;
    p.tiles_f = (int)((feats + ftile - 1) / ftile);
    p.tiles_t = (int)((tokens + TC_BN - 1) / TC_BN);
    p.status = status;
    p.ksplit = tc_ksplit(geo, dtype, transposed, tokens);
    if (p.ksplit > 1) {
        const size_t need = tc_ksplit_workspace_bytes(geo, dtype, transposed, tokens);
        if (!ws || ws_bytes < need) NMG_FAIL(NMG_ERR_WORKSPACE, "workspace of %zu bytes required for the partial tiles, got %zu", need, ws_bytes);
        p.partial = reinterpret_cast<float *>(((uintptr_t)ws + 255) & ~(uintptr_t)255);
        p.ld_partial = (int64_t)p.tiles_t * TC_BN;
    }
    const ProfileEvents pe = take_profile_events();
    if (pe.start) NMG_CUDA(cudaEventRecord(pe.start, st));
    rc = NMG_ERR_UNSUPPORTED;
#define NMG_TC_CASE(N_, M_)                                                                         \
    if (geo.n == N_ && geo.m == M_)                                                                \
        rc = tc_launch_nm<N_, M_>(dtype, transposed, p, tm, st);
    NMG_TC_CASE(1, 4)
    NMG_TC_CASE(2, 4)
    NMG_TC_CASE(1, 8)
    NMG_TC_CASE(2, 8)
    NMG_TC_CASE(1, 16)
#undef NMG_TC_CASE
    if (rc == NMG_ERR_UNSUPPORTED) set_error("no tensor-core kernel for %d:%d", geo.n, geo.m);
    if (rc == NMG_OK && p.ksplit > 1) {
        const int64_t plane = (int64_t)p.tiles_f * TC_BM * p.ld_partial;
        dim3 grid((unsigned)((tokens + 31) / 32), (unsigned)((feats + 31) / 32));
        if (grid.y > 65535) NMG_FAIL(NMG_ERR_UNSUPPORTED, "too many output features for the split-K reduction");
        if (dtype == NMG_F16)
            splitk_reduce_kernel<__half><<<grid, 256, 0, st>>>(p.partial, p.ksplit, plane, p.ld_partial, feats, tokens, static_cast<const __half *>(bias),
                                                                static_cast<__half *>(out), ld_out, out_token_major);
        else
            splitk_reduce_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(p.partial, p.ksplit, plane, p.ld_partial, feats, tokens,
                                                                       static_cast<const __nv_bfloat16 *>(bias), static_cast<__nv_bfloat16 *>(out), ld_out,
                                                                       out_token_major);
        NMG_CUDA(cudaGetLastError());
    }
    if (rc == NMG_OK && epi.any()) {
        const int64_t feats_out = transposed ? geo.K : geo.M;
        rc = out_token_major ? launch_epilogue(dtype, out, tokens, feats_out, ld_out, epi, st) : launch_epilogue(dtype, out, feats_out, tokens, ld_out, epi, st);
    }
    if (rc == NMG_OK && pe.stop) NMG_CUDA(cudaEventRecord(pe.stop, st));
    return rc;
}

// ---- activation / residual after kernels that do not fuse them --------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) epilogue_kernel(T *out, int64_t rows, int64_t cols, int64_t ld_out, int act, const T *res, int64_t ld_res) {
    for (int64_t r = blockIdx.y; r < rows; r += gridDim.y)
        for (int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; c < cols; c += (int64_t)gridDim.x * blockDim.x) {
            float v = DT<T>::to_f32(out[r * ld_out + c]);
            if (act == NMG_EPI_GELU) v = 0.5f * v * (1.f + erff(v * 0.70710678118654752f));
            if (res) v += DT<T>::to_f32(res[r * ld_res + c]);
            out[r * ld_out + c] = DT<T>::from_f32(v);
        }
}

int launch_epilogue(int dtype, void *out, int64_t rows, int64_t cols, int64_t ld_out, const Epilogue &epi, cudaStream_t st) {
    if (!epi.any() || rows < 1 || cols < 1) return NMG_OK;
    dim3 grid((unsigned)((cols + 255) / 256 < 64 ? (cols + 255) / 256 : 64), (unsigned)(rows < 65535 ? rows : 65535));
    NMG_DISPATCH_DTYPE(dtype, T, {
        epilogue_kernel<T><<<grid, 256, 0, st>>>(static_cast<T *>(out), rows, cols, ld_out, epi.act, static_cast<const T *>(epi.residual), epi.ld_res);
    });
    NMG_CUDA(cudaGetLastError());
    return NMG_OK;
}

}  // namespace nmg
