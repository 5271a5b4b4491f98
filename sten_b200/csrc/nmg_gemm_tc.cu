// Two-pass tensor-core matmul for large token counts: expand once, multiply at dense rate.
//
// The n:m blocks of the format run along the output-feature axis, so the tensor cores execute the dense product
// whatever the kernel does; what differs is how often a weight tile is expanded.  The fused kernel (nmg_spmm_tc.cu)
// expands every tile once per 256-token tile of the output, which costs about a third of its main loop; that is the
// right trade for few tokens, where the compressed weight is the HBM traffic.  With thousands of tokens it is cheaper
// to expand the weight ONCE into a transient dense 16-bit matrix in the caller's workspace (an HBM-bound pass of
// about 2.5 bytes per weight element) and run a plain TMA-fed tcgen05 matmul over it:
//
//   expand_dense_kernel   (val, idx) -> dense W [M][K] (forward) or W^T [K][M] (transposed product), 16-bit; fp32
//                         weights become three bf16 planes (exact hi / mid / lo split).  Works for every (n, m, g).
//   gemm_tc_kernel        persistent, one CTA per SM.  Warp 0 issues the TMA loads of both operands, warp 1 the
//                         MMAs (128 x 256 x 16, fp32 accumulators in TMEM), warps 2..9 drain accumulators.  16-bit
//                         mode double-buffers the accumulator (2 x 256 TMEM columns) so that the drain of one tile
//                         overlaps the MMAs of the next; fp32 mode uses the second half for the running sum into which
//                         the tensor core's partial tile is promoted every TC_CHUNK_KB k-blocks.
//
// All device-side waits are bounded: a wait that runs out sets the status word and the role leaves its loop; the
// CTA then meets at the common exit where TMEM is released.
#include <cstdlib>

#include "nmg_expand.cuh"
#include "nmg_spmm_simt.cuh"
#include "nmg_tc_common.cuh"

namespace nmg {

// =========================================================================================================
// Expansion pass
// =========================================================================================================
__device__ __forceinline__ void split3(float f, __nv_bfloat16 &hi, __nv_bfloat16 &mid, __nv_bfloat16 &lo) {
    hi = __float2bfloat16_rn(f);
    const float r1 = f - __bfloat162float(hi);
    mid = __float2bfloat16_rn(r1);
    lo = __float2bfloat16_rn(r1 - __bfloat162float(mid));
}

// Move `cnt` (1..8) consecutive elements of a shared-memory line to the destination planes and clear them in shared
// memory.  VEC: cnt == 8 and both sides are 16-byte aligned.
// PLAIN (fp32 only): the destination is an fp32 matrix, not three bf16 planes (the densifier's use of this pass).
template <typename T, bool VEC, bool PLAIN> __device__ __forceinline__ void expand_flush(const ExpandParams &p, T *line, int64_t off, int cnt) {
    if constexpr (sizeof(T) == 4 && PLAIN) {
        float *d = static_cast<float *>(p.dst) + off;
        if (VEC) {
            *reinterpret_cast<float4 *>(d) = *reinterpret_cast<const float4 *>(line);
            *reinterpret_cast<float4 *>(d + 4) = *reinterpret_cast<const float4 *>(line + 4);
            *reinterpret_cast<float4 *>(line) = make_float4(0.f, 0.f, 0.f, 0.f);
            *reinterpret_cast<float4 *>(line + 4) = make_float4(0.f, 0.f, 0.f, 0.f);
        } else {
            for (int i = 0; i < cnt; i++) { d[i] = line[i]; line[i] = 0.f; }
        }
    } else if constexpr (sizeof(T) == 2) {
        T *d = static_cast<T *>(p.dst) + off;
        if (VEC) {
            *reinterpret_cast<uint4 *>(d) = *reinterpret_cast<const uint4 *>(line);
            *reinterpret_cast<uint4 *>(line) = make_uint4(0, 0, 0, 0);
        } else {
            for (int i = 0; i < cnt; i++) { d[i] = line[i]; line[i] = DT<T>::from_f32(0.f); }
        }
    } else {
        __nv_bfloat16 *d = static_cast<__nv_bfloat16 *>(p.dst) + off;
        if (VEC) {
            const float4 a = *reinterpret_cast<const float4 *>(line), b = *reinterpret_cast<const float4 *>(line + 4);
            *reinterpret_cast<float4 *>(line) = make_float4(0.f, 0.f, 0.f, 0.f);
            *reinterpret_cast<float4 *>(line + 4) = make_float4(0.f, 0.f, 0.f, 0.f);
            const float f[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
            uint32_t w[3][4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                __nv_bfloat16 x[3], y[3];
                split3(f[2 * i], x[0], x[1], x[2]);
                split3(f[2 * i + 1], y[0], y[1], y[2]);
#pragma unroll
                for (int c = 0; c < 3; c++) w[c][i] = (uint32_t)__bfloat16_as_ushort(x[c]) | ((uint32_t)__bfloat16_as_ushort(y[c]) << 16);
            }
#pragma unroll
            for (int c = 0; c < 3; c++) *reinterpret_cast<uint4 *>(d + c * p.plane_elems) = make_uint4(w[c][0], w[c][1], w[c][2], w[c][3]);
        } else {
            for (int i = 0; i < cnt; i++) {
                __nv_bfloat16 x[3];
                split3(line[i], x[0], x[1], x[2]);
                line[i] = 0.f;
                for (int c = 0; c < 3; c++) d[c * p.plane_elems + i] = x[c];
            }
        }
    }
}

// Work item = (column chunk kc, R consecutive row-blocks).  The item's dense tile lives in shared memory, in the
// orientation of the destination (TR = false: lines are weight rows, cc columns long; TR = true: lines are weight
// columns, R * m rows long).  It starts as zeros; the item's non-zeros are scattered into it straight from global
// memory (coalesced reads of val and idx, one thread per slot), and the tile is then moved out with 16-byte accesses
// that also restore the zeros.
// N_ = n for the vectorised scatter (1 or 2), 0 for the generic one.
template <typename T, bool TR, int N_, bool PLAIN = false>
__global__ void __launch_bounds__(EXPAND_THREADS) expand_dense_kernel(const ExpandParams prm) {
    extern __shared__ __align__(16) char smem[];
    constexpr bool VEC_OK = N_ > 0;
    const int n = N_ > 0 ? N_ : prm.n, m = prm.m, g = prm.g, cc = prm.cc, R = prm.R, pitch = prm.pitch;
    const int lines = TR ? cc : R * m;
    T *tile = reinterpret_cast<T *>(smem);                                  // [lines][pitch]
    int8_t *ord = reinterpret_cast<int8_t *>(tile + (size_t)lines * pitch);  // [C][n]
    // The matmul kernel that follows is launched with programmatic stream serialization: it may become resident and run
    // its prologue while this grid drains, and reads nothing this grid writes before its griddepcontrol.wait.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    for (int i = threadIdx.x; i < prm.C * n; i += EXPAND_THREADS) ord[i] = prm.order[i];
    for (int i = threadIdx.x; i < lines * pitch; i += EXPAND_THREADS) tile[i] = DT<T>::from_f32(0.f);

    const T *val = static_cast<const T *>(prm.val);
    const int64_t groups = (prm.nb + R - 1) / R;
    const int64_t items = groups * prm.nc;
    const int vec_per_line = pitch / 8;  // pitch is a multiple of 8

    for (int64_t item = blockIdx.x; item < items; item += gridDim.x) {
        const int64_t kc = item / groups, mb0 = (item - kc * groups) * R;
        const int rj = (int)(prm.nb - mb0 < R ? prm.nb - mb0 : R);  // row-blocks in this item
        __syncthreads();  // the tile is all zeros again
        expand_scatter_item<T, TR, N_>(prm, tile, ord, kc, mb0, rj);
        __syncthreads();
        const int64_t col0 = kc * cc, r0 = mb0 * m;
        // line l, elements e .. e+7 -> dst[(TR ? col0 + l : r0 + l)][(TR ? r0 : col0) + e]
        const int64_t line_lim = TR ? prm.K - col0 : prm.M - r0;   // lines inside the weight
        const int64_t elem_lim = TR ? prm.M - r0 : prm.K - col0;   // elements of a line inside the weight
        const int ne = TR ? rj * m : cc;                            // elements of a line this item owns
        const bool aligned = ((TR ? r0 : col0) % 8) == 0;           // ld is a multiple of 8, the workspace is 256-byte aligned
        for (int v = threadIdx.x; v < lines * vec_per_line; v += EXPAND_THREADS) {
            const int l = v / vec_per_line, e = (v - l * vec_per_line) * 8;
            T *line = tile + l * pitch + e;
            if (l >= line_lim || e >= ne || e >= elem_lim) {  // outside the weight: nothing to store, but keep the tile clean
                if constexpr (sizeof(T) == 2) *reinterpret_cast<uint4 *>(line) = make_uint4(0, 0, 0, 0);
                else { *reinterpret_cast<float4 *>(line) = make_float4(0.f, 0.f, 0.f, 0.f); *reinterpret_cast<float4 *>(line + 4) = make_float4(0.f, 0.f, 0.f, 0.f); }
                continue;
            }
            const int64_t off = ((TR ? col0 : r0) + l) * prm.ld + (TR ? r0 : col0) + e;
            // A full vector may run past the item's elements only into the row's padding (last chunk / last group:
            // ld = round_up(extent, 8)), never into elements another item owns.
            if (aligned && (e + 8 <= ne || ne >= elem_lim)) {
                expand_flush<T, true, PLAIN>(prm, line, off, 8);
            } else {
                int cnt = ne - e < 8 ? ne - e : 8;
                if (elem_lim - e < cnt) cnt = (int)(elem_lim - e);
                expand_flush<T, false, PLAIN>(prm, line, off, cnt);
                // elements of the vector past cnt were never written by this item's valid slots; clear them anyway
                for (int i = cnt; i < 8; i++) line[i] = DT<T>::from_f32(0.f);
            }
        }
    }
}

static int expand_pitch(const Geo &geo, bool tr, int R) { return (int)round_up(tr ? (int64_t)R * geo.m : (int64_t)geo.cc, 8) + 8; }
static size_t expand_smem_bytes(const Geo &geo, size_t es, bool tr, int R) {
    const size_t lines = tr ? (size_t)geo.cc : (size_t)R * geo.m;
    return lines * expand_pitch(geo, tr, R) * es + (size_t)geo.C * geo.n + 16;
}
static int expand_rows_per_item(const Geo &geo, size_t es, bool tr) {
    int R = 64 / geo.m;
    if (R < 1) R = 1;
    while (R > 1 && expand_smem_bytes(geo, es, tr, R) > 64 * 1024) R >>= 1;
    return R;
}

// =========================================================================================================
// Dense-operand matmul
// =========================================================================================================
constexpr int GEMM_DRAIN_WARPS = 8;   // two per TMEM lane quarter, each takes half of the accumulator's columns
constexpr int GEMM_THREADS = 32 * (2 + GEMM_DRAIN_WARPS);  // TMA warp, MMA warp, drain warps
constexpr int GEMM_RING_BYTES = TC_STAGES * (TC_A_BYTES + TC_B_BYTES);  // 192 KB of operand stages in either mode

constexpr int GEMM_MAX_OUTS = 8;
struct GemmParams {
    const void *bias;  // [out_feats] or NULL
    void *outs[GEMM_MAX_OUTS];  // the result is written to every one of these (same shape and pitch): outs[0] is the
    int n_out;                  // caller's buffer, the others are typically the same buffer on peer GPUs
    void *mc_out;               // NVSwitch multicast address mapping onto all of outs[], or NULL: one multimem.st reaches every GPU
    const void *residual;       // added after the activation, same orientation as the output, or NULL
    int64_t ld_res;
    int act;                    // NMG_EPI_NONE / NMG_EPI_GELU applied to (product + bias)
    int bias_cols;              // bias runs along the accumulator's columns ("tokens" below) instead of its rows
    int out_tma;                // staged output with one destination: the staging tile leaves as one tiled bulk store per group
    int res_vec;                // staged output: the residual is read in the same 16-byte pieces as the output is written
    int64_t out_feats, red, ntok, ld_out;
    int out_token_major;
    int out_staged;    // feature-major output whose rows are 16-byte aligned: go through the staging tile
    int out_tm_vec;    // token-major output (and residual) whose rows are 16-byte aligned: transposed in the staging tile, 16-byte stores
    int tiles_f, tiles_t;  // tiles_f counts tiles of 128 features (one CTA per tile) or 256 (CTA pairs)
    int band;              // width of the tile order's bands, in feature tiles
    unsigned *wave_ctr;    // zeroed counter for the producers' soft rendezvous before every tile, or NULL
    int *status;
};
constexpr int GEMM_STAGING_BYTES = GEMM_DRAIN_WARPS * 4096;  // per drain warp: 32 feature rows x 128 bytes

struct GemmMaps {
    CUtensorMap a[3];  // weight planes, box 64 x 128, 128-byte swizzle
    CUtensorMap b[3];  // activation planes, box 64 x 256 (64 x 128 for CTA pairs)
    CUtensorMap out;   // out_tma: the output, box 128 bytes x 32 rows, 128-byte swizzle
};

// Exact (erf) GELU with a short erf: erf(x) = 1 - (a1 t + ... + a5 t^5) exp(-x^2), t = 1 / (1 + p x) for x >= 0 (Abramowitz &
// Stegun 7.1.26, absolute error 1.5e-7, i.e. below fp32 rounding of the result for |v| of order one).  With x = |v| / sqrt(2)
// and v * sign(v) = |v|, gelu(v) = v (1 + erf(v / sqrt 2)) / 2 collapses to max(v, 0) - |v| q(t) 2^(-v^2 log2(e) / 2) where q
// carries the halved coefficients: fourteen instructions, two of them on the special-function unit (flush-to-zero forms, which
// need no range fix-up), against the library erf's thirty.  The drain warps apply it to 128 x 256 values per tile.
__device__ __forceinline__ float gelu_erf(float v) {
    const float av = fabsf(v);
    float t, e;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(t) : "f"(fmaf(0.23164189f, av, 1.f)));   // p / sqrt(2)
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"((v * -0.72134752f) * v));          // log2(e) / 2
    const float q = fmaf(fmaf(fmaf(fmaf(0.5307027145f, t, -0.7265760135f), t, 0.7107068705f), t, -0.142248368f), t, 0.127414796f) * t;
    return fmaf(-(av * q), e, fmaxf(v, 0.f));
}

// PAIR = false: one CTA per 128-feature x 256-token tile.
// PAIR = true (16-bit operands): two CTAs of a cluster share a 256-feature x 256-token tile.  Each loads the weight rows
// of its own 128 features and only half of the activation tile (128 tokens); the MMA (cta_group::2, M = 256, issued by the
// even CTA) reads both halves from both shared memories.  An SM then takes in 32 KB per 64 reduction elements instead of
// 48 KB, which is what keeps the tensor core fed from L2.  full[s] lives in the even ("leader") CTA and receives the TMA
// bytes of both; empty[s] and acc_full[b] exist in both CTAs and are signalled by multicast commits; acc_free[b] lives in
// the leader and collects the drain warps of both CTAs.  No load is multicast.
// TMA_OUT = true: the one-destination staged output, leaving as tiled bulk stores; only that output path is compiled,
// which keeps the drain warps' code and register needs small.  TMA_OUT = false: every other output form.
template <typename T, bool PAIR, bool TMA_OUT>
__global__ void __launch_bounds__(GEMM_THREADS, 1) gemm_tc_kernel(const GemmParams prm, const __grid_constant__ GemmMaps maps) {
    constexpr int TERMS = TcMode<T>::TERMS;
    using E = typename TcMode<T>::elem;
    constexpr bool SPLIT = TERMS > 1;
    static_assert(!(PAIR && SPLIT), "CTA pairs serve the 16-bit mode");
    constexpr int NBUF = SPLIT ? 1 : 2;  // accumulator tiles in flight between the MMA issuer and the drain warps
    constexpr uint32_t TMEM_COLS = 2 * TC_ACC_COLS;
    constexpr int B_BYTES = PAIR ? TC_B_BYTES / 2 : TC_B_BYTES;
    constexpr int STAGE_BYTES = TC_A_BYTES + B_BYTES;
    constexpr int STAGES = GEMM_RING_BYTES / STAGE_BYTES;  // 4, or 6 for pairs
    constexpr int TILE_FEATS = PAIR ? 2 * TC_BM : TC_BM;

    extern __shared__ char smem_raw[];
    char *smem = reinterpret_cast<char *>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    char *staging = smem + GEMM_RING_BYTES;
    char *misc = staging + GEMM_STAGING_BYTES;
    uint64_t *full = reinterpret_cast<uint64_t *>(misc);   // pairs: meaningful in the leader only
    uint64_t *empty = full + STAGES;
    uint64_t *acc_full = empty + STAGES;  // [2] MMA issuer -> drain warps: unit complete in accumulator b
    uint64_t *acc_free = acc_full + 2;    // [2] drain warps -> MMA issuer: accumulator b may be overwritten (pairs: leader only)
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(misc + 192);
    static_assert((2 * STAGES + 4) * 8 <= 192, "barrier block too small");

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
    const bool leader = rank == 0;
    const int unit_id = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;      // CTA (or pair) index
    const int nunits = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
    // A "unit" is what the MMA issuer hands to the drain warps: a whole tile (16-bit) or a chunk of k-blocks (fp32).
    const int ntiles = prm.tiles_f * prm.tiles_t;
    const int my_tiles = (unit_id < ntiles) ? (ntiles - unit_id + nunits - 1) / nunits : 0;
    const int nkb = (int)((prm.red + TC_BK - 1) / TC_BK) * TERMS;  // iterations per tile: k-blocks x split terms (term fastest)
    const int chunk_it = SPLIT ? TC_CHUNK_KB * TERMS : nkb;
    const int nchunks = (nkb + chunk_it - 1) / chunk_it;

    if (tid == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_free[b], GEMM_DRAIN_WARPS * (PAIR ? 2 : 1));  // lane 0 of each drain warp (of both CTAs)
        }
        mbar_fence_init();
    }
    if (warp == 1) {
        if constexpr (PAIR) tmem_alloc_pair(tmem_slot, TMEM_COLS);
        else tmem_alloc(tmem_slot, TMEM_COLS);
    }
    tc_fence_before();
    __syncthreads();
    if constexpr (PAIR) cluster_sync_all();  // barriers of both CTAs are initialised before anyone arrives remotely
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t full_leader = PAIR ? map_to_rank(smem_u32(&full[0]), 0) : 0u;
    const uint32_t acc_free_leader = PAIR ? map_to_rank(smem_u32(&acc_free[0]), 0) : 0u;

    auto wait = [&](uint64_t *bar, uint32_t parity, int code) -> bool {
        if constexpr (PAIR) return mbar_wait_cluster_bounded(bar, parity, prm.status, code);
        else return mbar_wait_bounded(bar, parity, prm.status, code);
    };
    auto tile_origin = [&](int ti, int &feat0, int &tok0) {  // feat0: first feature of THIS CTA's 128 rows
        int tile_f, tile_t;
        tile_of_cta(unit_id + ti * nunits, prm.tiles_f, prm.tiles_t, tile_f, tile_t, prm.band);
        feat0 = tile_f * TILE_FEATS + (int)rank * TC_BM;
        tok0 = tile_t * TC_BN;
    };

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (one lane per CTA)
        if (lane == 0) {
            int it = 0;
            bool ok = true;
            // Everything this kernel reads that an earlier kernel of the stream wrote (the expanded weight, the
            // activations) arrives through the loads below: wait here for the preceding grid to complete and flush.
            asm volatile("griddepcontrol.wait;" ::: "memory");
            unsigned arrivals = 0;
            for (int ti = 0; ti < my_tiles && ok; ti++) {
                int feat0, tok0;
                tile_origin(ti, feat0, tok0);
                if (prm.wave_ctr && ti > 0) {
                    // CTAs whose tiles share operand panels read them from HBM once only while they stream through the
                    // reduction in step; left alone they drift apart over the waves (measured: 2.2 MB of DRAM reads per
                    // 256 x 256 x 16384 tile in the first dozen waves, 3.9 MB averaged over 55).  So the producers meet,
                    // softly, before each tile: everyone that has a tile ti counts in.
                    const int left = ntiles - ti * nunits;
                    arrivals += (unsigned)((left < nunits ? left : nunits) * (PAIR ? 2 : 1));
                    soft_rendezvous(prm.wave_ctr, arrivals, (uint64_t)nkb * 40);
                }
                for (int kb = 0; kb < nkb; kb++, it++) {
                    const int s = it % STAGES;
                    const uint32_t ph = (uint32_t)((it / STAGES) & 1);
                    if (!(ok = wait(&empty[s], ph ^ 1, 21))) break;
                    const int term = kb % TERMS;
                    const int wc = TERMS == 1 ? 0 : kSplitW[term], xc = TERMS == 1 ? 0 : kSplitX[term];
                    char *stage = smem + s * STAGE_BYTES;
                    if constexpr (PAIR) {
                        if (leader) mbar_expect_tx(&full[s], 2 * STAGE_BYTES);  // both CTAs report to this barrier
                        tma_load_2d_pair(stage, &maps.a[wc], (kb / TERMS) * TC_BK, feat0, full_leader + s * 8);
                        tma_load_2d_pair(stage + TC_A_BYTES, &maps.b[xc], (kb / TERMS) * TC_BK, tok0 + (int)rank * 128, full_leader + s * 8);
                    } else {
                        mbar_expect_tx(&full[s], STAGE_BYTES);
                        tma_load_2d(stage, &maps.a[wc], (kb / TERMS) * TC_BK, feat0, &full[s]);
                        tma_load_2d(stage + TC_A_BYTES, &maps.b[xc], (kb / TERMS) * TC_BK, tok0, &full[s]);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (one lane; of the leader for pairs)
        if (lane == 0 && leader) {
            uint32_t idesc = make_idesc<E>();
            if constexpr (PAIR) idesc = (idesc & ~(0x1fu << 24)) | ((uint32_t)(256 >> 4) << 24);  // M = 256 across the pair
            bool ok = true;
            int it = 0, unit = 0;
            for (int ti = 0; ti < my_tiles && ok; ti++) {
                int kb = 0;
                for (int c = 0; c < nchunks && ok; c++, unit++) {
                    const int b = unit % NBUF, use = unit / NBUF;
                    if (use > 0) ok = wait(&acc_free[b], (uint32_t)((use - 1) & 1), 26);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t d_tmem = tmem_base + (uint32_t)(b * TC_ACC_COLS);
                    const int kend = (kb + chunk_it < nkb) ? kb + chunk_it : nkb;
                    for (bool first = true; kb < kend; kb++, it++, first = false) {
                        const int s = it % STAGES;
                        const uint32_t ph = (uint32_t)((it / STAGES) & 1);
                        if (!(ok = wait(&full[s], ph, 22))) break;
                        tc_fence_after();
                        const uint64_t adesc = make_sw128_desc(smem_u32(smem + s * STAGE_BYTES));
                        const uint64_t bdesc = make_sw128_desc(smem_u32(smem + s * STAGE_BYTES + TC_A_BYTES));
#pragma unroll
                        for (int k = 0; k < TC_BK / 16; k++) {  // 16 elements = 32 bytes = 2 descriptor units per step
                            if constexpr (PAIR) tc2_mma_f16(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (first && k == 0) ? 0u : 1u);
                            else tc_mma_f16(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (first && k == 0) ? 0u : 1u);
                        }
                        if constexpr (PAIR) tc2_commit_both(&empty[s]);
                        else tc_commit(&empty[s]);  // arrives when the MMAs above have read the stage
                    }
                    // arrives when the unit's MMAs have written TMEM (also on the error path)
                    if constexpr (PAIR) tc2_commit_both(&acc_full[b]);
                    else tc_commit(&acc_full[b]);
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ drain warps: promotion and epilogue
        // Feature-major output (out[feature][token]) leaves through a per-warp staging tile: the warp's 32 features x
        // 128 bytes of tokens, 16-byte chunks XOR-swizzled by row.  TMEM hands every lane one feature row; the staging
        // tile turns that into stores whose 8 neighbouring lanes cover 128 contiguous bytes of one output row, which
        // is what both HBM and NVLink want, and the same registers are stored to every destination buffer.
        constexpr int CHUNK_TOK = 16 / (int)sizeof(T);         // tokens per 16-byte chunk
        constexpr int GROUP_TOK = 128 / (int)sizeof(T);        // tokens per staged row: 64 (16-bit) or 32 (fp32)
        constexpr int GROUP_SLICES = GROUP_TOK / 32;           // 32-column TMEM slices per staged group
        constexpr bool RES_AHEAD = TMA_OUT && sizeof(T) == 2;  // residual fetched one slice ahead (fp32 rows would take 2 x 32 registers)
        constexpr int RQ = RES_AHEAD ? 4 : 1;                  // 16-byte pieces of one slice row of the residual
        const int q = warp & 3;  // TMEM lane quarter this warp may access
        constexpr int SLICES = (TC_BN / 32) / (GEMM_DRAIN_WARPS / 4);  // 32-column slices per warp
        const int sl0 = ((warp - 2) >> 2) * SLICES;                    // this warp's first slice
        const uint32_t lane_base = tmem_base + ((uint32_t)(q * 32) << 16);
        char *stage_w = staging + (warp - 2) * 4096;
        const T *res = static_cast<const T *>(prm.residual);
        const bool gelu = prm.act == NMG_EPI_GELU;
        // The bias and the residual are read with ordinary loads, possibly before the first accumulator is ready: like the
        // producer's loads they must not run ahead of the grid this one was launched behind.
        asm volatile("griddepcontrol.wait;" ::: "memory");
        int unit = 0;
        bool ok = true;
        for (int ti = 0; ti < my_tiles && ok; ti++) {
            int feat0, tok0;
            tile_origin(ti, feat0, tok0);
            const int64_t feat = (int64_t)feat0 + q * 32 + lane;
            const bool feat_ok = feat < prm.out_feats;
            const float bias = (prm.bias && !prm.bias_cols && feat_ok) ? DT<T>::to_f32(static_cast<const T *>(prm.bias)[feat]) : 0.f;
            // column bias: lane l keeps the value of column l of each of this warp's slices; the slice's loop fetches
            // element j's value from lane j
            float bcol[SLICES];
#pragma unroll
            for (int i = 0; i < SLICES; i++) {
                const int64_t col = (int64_t)tok0 + (sl0 + i) * 32 + lane;
                bcol[i] = (prm.bias && prm.bias_cols && col < prm.ntok) ? DT<T>::to_f32(static_cast<const T *>(prm.bias)[col]) : 0.f;
            }
            // The residual of a slice (this lane's row, 32 elements) is fetched in 16-byte pieces one slice ahead of its
            // use, like the accumulator, when the bulk-store path runs and the residual's rows allow it.
            auto res_vec_ok = [&](int64_t tokc) -> bool { return TMA_OUT && prm.res_vec && tokc + 32 <= prm.ntok; };
            auto res_fetch = [&](int sl, uint4 (&qr)[RQ]) {
                if constexpr (RES_AHEAD) {
                    const int64_t tokc = (int64_t)tok0 + sl * 32;
                    if (res && feat_ok && res_vec_ok(tokc)) {
#pragma unroll
                        for (int v = 0; v < RQ; v++) qr[v] = __ldg(reinterpret_cast<const uint4 *>(res + feat * prm.ld_res + tokc) + v);
                    }
                }
            };
            for (int c = 0; c < nchunks; c++, unit++) {
                const int b = unit % NBUF, use = unit / NBUF;
                if (!(ok = wait(&acc_full[b], (uint32_t)(use & 1), 25))) break;
                tc_fence_after();
                const bool last = c == nchunks - 1;
                auto release = [&]() {  // this warp's TMEM reads of the unit are done: the issuer may reuse the accumulator once all warps say so
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        if constexpr (PAIR) mbar_arrive_remote(acc_free_leader + b * 8);
                        else mbar_arrive(&acc_free[b]);
                    }
                };
                // handle(sl, r, qr): slice sl of the unit is in registers r (this lane's feature row, 32 tokens); qr holds the
                // same 32 elements of the residual when res_fetch found them loadable in 16-byte pieces
                auto handle = [&](int sl, uint32_t (&r)[32], const uint4 (&qr)[RQ]) {
                    if (SPLIT && c > 0) {
                        uint32_t run[32];
                        tmem_ld32(lane_base + (uint32_t)(TC_ACC_COLS + sl * 32), run);
#pragma unroll
                        for (int j = 0; j < 32; j++) r[j] = __float_as_uint(__fadd_rn(__uint_as_float(run[j]), __uint_as_float(r[j])));
                    }
                    if (!last) {
                        tmem_st32(lane_base + (uint32_t)(TC_ACC_COLS + sl * 32), r);
                        return;
                    }
                    if (sl == sl0 + SLICES - 1) release();
                    const int64_t tokc = (int64_t)tok0 + sl * 32;
                    // activation(product + bias), kept as fp32 bits in r.  The activation sits in one warp-uniform branch
                    // around its own unrolled loop: the 32 evaluations are independent and interleave, where a test per
                    // element would run them one after the other at full dependent latency.
                    if (prm.bias_cols) {
                        float bc = bcol[0];
#pragma unroll
                        for (int i = 1; i < SLICES; i++) bc = (sl - sl0 == i) ? bcol[i] : bc;
#pragma unroll
                        for (int j = 0; j < 32; j++) r[j] = __float_as_uint(__uint_as_float(r[j]) + __shfl_sync(0xffffffffu, bc, j));
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j++) r[j] = __float_as_uint(__uint_as_float(r[j]) + bias);
                    }
                    if (gelu) {
#pragma unroll
                        for (int j = 0; j < 32; j++) r[j] = __float_as_uint(gelu_erf(__uint_as_float(r[j])));
                    }
                    if constexpr (TMA_OUT) {
                        if (res && feat_ok) {
                            if (res_vec_ok(tokc)) {
                                if constexpr (RES_AHEAD) {
                                    const T *e = reinterpret_cast<const T *>(qr);
#pragma unroll
                                    for (int j = 0; j < 32; j++) r[j] = __float_as_uint(__uint_as_float(r[j]) + DT<T>::to_f32(e[j]));
                                } else {
                                    const uint4 *src = reinterpret_cast<const uint4 *>(res + feat * prm.ld_res + tokc);
#pragma unroll
                                    for (int v = 0; v < 8; v++) {
                                        const uint4 w = __ldg(src + v);
                                        r[4 * v] = __float_as_uint(__uint_as_float(r[4 * v]) + __uint_as_float(w.x));
                                        r[4 * v + 1] = __float_as_uint(__uint_as_float(r[4 * v + 1]) + __uint_as_float(w.y));
                                        r[4 * v + 2] = __float_as_uint(__uint_as_float(r[4 * v + 2]) + __uint_as_float(w.z));
                                        r[4 * v + 3] = __float_as_uint(__uint_as_float(r[4 * v + 3]) + __uint_as_float(w.w));
                                    }
                                }
                            } else {
                                for (int j = 0; j < 32; j++)
                                    if (tokc + j < prm.ntok) r[j] = __float_as_uint(__uint_as_float(r[j]) + DT<T>::to_f32(res[feat * prm.ld_res + tokc + j]));
                            }
                        }
                        // registers -> staging row `lane` (16-byte chunks XOR-swizzled by row: the 128-byte swizzle of the
                        // output's tensor map), once the previous group's bulk store has read the tile
                        constexpr int CH = 32 / CHUNK_TOK;  // chunks per slice: 4 (16-bit) or 8 (fp32)
                        const int ch0 = (sl % GROUP_SLICES) * CH;
                        if ((sl % GROUP_SLICES) == 0) {
                            if (lane == 0) tma_store_wait_read();
                            __syncwarp();
                        }
#pragma unroll
                        for (int v = 0; v < CH; v++) {
                            uint4 w;
                            if constexpr (sizeof(T) == 4) {
                                w = make_uint4(r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]);
                            } else {  // one packed conversion per pair
                                w = make_uint4(pack2<T>(__uint_as_float(r[8 * v]), __uint_as_float(r[8 * v + 1])),
                                               pack2<T>(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3])),
                                               pack2<T>(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5])),
                                               pack2<T>(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7])));
                            }
                            *reinterpret_cast<uint4 *>(stage_w + lane * 128 + (((ch0 + v) ^ (lane & 7)) << 4)) = w;
                        }
                        if ((sl % GROUP_SLICES) != GROUP_SLICES - 1) return;
                        // The staging tile is exactly one swizzled box of 32 rows x 128 bytes: hand it to the copy engine,
                        // which clips it at the tensor's edges, and go on with the next slice.
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0) tma_store_2d(&maps.out, stage_w, tok0 + (sl / GROUP_SLICES) * GROUP_TOK, feat0 + q * 32);
                        return;
                    } else {
                    if (prm.out_tm_vec) {
                        // Token-major output through the staging tile.  TMEM hands every lane one feature and 32 tokens;
                        // out[token][feature] wants neighbouring lanes on neighbouring features, which scalar stores
                        // give only 2 bytes at a time.  The slice is transposed in shared memory ([token][32 features])
                        // and leaves -- after the residual, fetched in the same 16-byte pieces before the transposition
                        // so that its latency is covered, is added -- in 16-byte stores.
                        constexpr int CPR = 32 * (int)sizeof(T) / 16;  // 16-byte chunks per staged row: 4 (16-bit) or 8 (fp32)
                        const int64_t fbase = (int64_t)feat0 + q * 32 + (lane % CPR) * CHUNK_TOK;  // CHUNK_TOK = elements per chunk
                        const bool whole = fbase + CHUNK_TOK <= prm.out_feats;
                        uint4 rv[CPR];
                        if (res) {
#pragma unroll
                            for (int i = 0; i < CPR; i++) {
                                const int64_t tok = tokc + i * (32 / CPR) + lane / CPR;
                                rv[i] = make_uint4(0u, 0u, 0u, 0u);
                                if (tok < prm.ntok && whole) rv[i] = __ldg(reinterpret_cast<const uint4 *>(res + tok * prm.ld_res + fbase));
                            }
                        }
                        T *st = reinterpret_cast<T *>(stage_w);
#pragma unroll
                        for (int j = 0; j < 32; j++) st[j * 32 + lane] = DT<T>::from_f32(__uint_as_float(r[j]));
                        __syncwarp();
#pragma unroll
                        for (int i = 0; i < CPR; i++) {
                            const int row = i * (32 / CPR) + lane / CPR;
                            const int64_t tok = tokc + row;
                            if (tok >= prm.ntok || fbase >= prm.out_feats) continue;
                            uint4 w = *reinterpret_cast<const uint4 *>(stage_w + row * 32 * (int)sizeof(T) + (lane % CPR) * 16);
                            if (res) {
                                __align__(16) T a[CHUNK_TOK], b[CHUNK_TOK];
                                *reinterpret_cast<uint4 *>(a) = w;
                                *reinterpret_cast<uint4 *>(b) = rv[i];
                                if (!whole)  // ragged end of the feature axis
                                    for (int k = 0; k < CHUNK_TOK; k++) b[k] = fbase + k < prm.out_feats ? res[tok * prm.ld_res + fbase + k] : DT<T>::from_f32(0.f);
#pragma unroll
                                for (int k = 0; k < CHUNK_TOK; k++) a[k] = DT<T>::from_f32(DT<T>::to_f32(a[k]) + DT<T>::to_f32(b[k]));
                                w = *reinterpret_cast<const uint4 *>(a);
                            }
                            T *dst = static_cast<T *>(prm.outs[0]) + tok * prm.ld_out + fbase;
                            if (whole) *reinterpret_cast<uint4 *>(dst) = w;
                            else {
                                const T *e = reinterpret_cast<const T *>(&w);
                                for (int k = 0; k < CHUNK_TOK && fbase + k < prm.out_feats; k++) dst[k] = e[k];
                            }
                        }
                        __syncwarp();  // the staging rows are free for the next slice
                        return;
                    }
                    // the other output forms take the residual element by element, again under one uniform branch
                    const bool res_late = prm.out_staged && prm.res_vec;
                    if (res && feat_ok && !res_late) {
                        if (prm.out_token_major) {
#pragma unroll
                            for (int j = 0; j < 32; j++)
                                if (tokc + j < prm.ntok) r[j] = __float_as_uint(__uint_as_float(r[j]) + DT<T>::to_f32(res[(tokc + j) * prm.ld_res + feat]));
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; j++)
                                if (tokc + j < prm.ntok) r[j] = __float_as_uint(__uint_as_float(r[j]) + DT<T>::to_f32(res[feat * prm.ld_res + tokc + j]));
                        }
                    }
                    if (!prm.out_staged) {
                        if (tokc >= prm.ntok || !feat_ok) return;
                        if (prm.out_token_major && prm.n_out == 1 && tokc + 32 <= prm.ntok) {
                            // full slice of the F.linear layout: one conversion, one pointer step and one store per element
                            T *p = static_cast<T *>(prm.outs[0]) + tokc * prm.ld_out + feat;
#pragma unroll
                            for (int j = 0; j < 32; j++, p += prm.ld_out) *p = DT<T>::from_f32(__uint_as_float(r[j]));
                            return;
                        }
                        for (int d = 0; d < prm.n_out; d++) {
                            T *out = static_cast<T *>(prm.outs[d]);
#pragma unroll
                            for (int j = 0; j < 32; j++) {
                                const int64_t tok = tokc + j;
                                if (tok < prm.ntok) {
                                    const T o = DT<T>::from_f32(__uint_as_float(r[j]));
                                    if (prm.out_token_major) out[tok * prm.ld_out + feat] = o;
                                    else out[feat * prm.ld_out + tok] = o;
                                }
                            }
                        }
                        return;
                    }
                    // registers -> staging row `lane`
                    constexpr int CH = 32 / CHUNK_TOK;  // chunks per slice: 4 (16-bit) or 8 (fp32)
                    const int ch0 = (sl % GROUP_SLICES) * CH;
#pragma unroll
                    for (int v = 0; v < CH; v++) {
                        uint4 w;
                        if constexpr (sizeof(T) == 4) {
                            w = make_uint4(r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]);
                        } else {  // one packed conversion per pair
                            w = make_uint4(pack2<T>(__uint_as_float(r[8 * v]), __uint_as_float(r[8 * v + 1])),
                                           pack2<T>(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3])),
                                           pack2<T>(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5])),
                                           pack2<T>(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7])));
                        }
                        *reinterpret_cast<uint4 *>(stage_w + lane * 128 + (((ch0 + v) ^ (lane & 7)) << 4)) = w;
                    }
                    if ((sl % GROUP_SLICES) != GROUP_SLICES - 1) return;
                    __syncwarp();
                    // staging -> every destination: lane handles chunk (lane & 7) of rows (lane >> 3) + 4 i
                    const int64_t tokg = (int64_t)tok0 + (sl / GROUP_SLICES) * GROUP_TOK + (lane & 7) * CHUNK_TOK;
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        const int row = i * 4 + (lane >> 3);
                        const int64_t f = (int64_t)feat0 + q * 32 + row;
                        if (f >= prm.out_feats || tokg >= prm.ntok) continue;
                        uint4 w = *reinterpret_cast<const uint4 *>(stage_w + row * 128 + (((lane & 7) ^ (row & 7)) << 4));
                        if (res && res_late) {  // the loads of the eight rows are independent of one another and of the staging tile
                            __align__(16) T a[CHUNK_TOK], b[CHUNK_TOK];
                            *reinterpret_cast<uint4 *>(a) = w;
                            if (tokg + CHUNK_TOK <= prm.ntok) *reinterpret_cast<uint4 *>(b) = __ldg(reinterpret_cast<const uint4 *>(res + f * prm.ld_res + tokg));
                            else
                                for (int k = 0; k < CHUNK_TOK; k++) b[k] = tokg + k < prm.ntok ? res[f * prm.ld_res + tokg + k] : DT<T>::from_f32(0.f);
#pragma unroll
                            for (int k = 0; k < CHUNK_TOK; k++) a[k] = DT<T>::from_f32(DT<T>::to_f32(a[k]) + DT<T>::to_f32(b[k]));
                            w = *reinterpret_cast<const uint4 *>(a);
                        }
                        if (tokg + CHUNK_TOK <= prm.ntok) {
                            if (prm.mc_out) {  // the switch replicates the 16 bytes to every GPU of the multicast group
                                multimem_st_v4(static_cast<T *>(prm.mc_out) + f * prm.ld_out + tokg, w);
                                continue;
                            }
                            for (int d = 0; d < prm.n_out; d++)
                                *reinterpret_cast<uint4 *>(static_cast<T *>(prm.outs[d]) + f * prm.ld_out + tokg) = w;
                        } else {  // ragged end of the token axis
                            const T *e = reinterpret_cast<const T *>(&w);
                            for (int d = 0; d < prm.n_out; d++)
                                for (int k = 0; k < CHUNK_TOK && tokg + k < prm.ntok; k++)
                                    (static_cast<T *>(prm.outs[d]) + f * prm.ld_out + tokg)[k] = e[k];
                        }
                    }
                    __syncwarp();  // the staging rows are free for the next group
                    }  // !TMA_OUT
                };
                // TMEM reads are software-pipelined: the load of the next slice is in flight while this one is converted
                // and stored; tmem_ld_fence ties the wait to the registers so no use can move above it.
                uint32_t ra[32], rb[32];
                uint4 qa[RQ], qb[RQ];
                const uint32_t acc_addr = lane_base + (uint32_t)(b * TC_ACC_COLS);
                tmem_ld32_issue(acc_addr + (uint32_t)(sl0 * 32), ra);
                if (last) res_fetch(sl0, qa);
#pragma unroll 1
                for (int sl = sl0; sl < sl0 + SLICES; sl += 2) {
                    tmem_ld_fence(ra);
                    tmem_ld32_issue(acc_addr + (uint32_t)((sl + 1) * 32), rb);
                    if (last) res_fetch(sl + 1, qb);
                    handle(sl, ra, qa);
                    tmem_ld_fence(rb);
                    if (sl + 2 < sl0 + SLICES) {
                        tmem_ld32_issue(acc_addr + (uint32_t)((sl + 2) * 32), ra);
                        if (last) res_fetch(sl + 2, qa);
                    }
                    handle(sl + 1, rb, qb);
                }
                if (!last) release();  // promotion finished: hand the accumulator back
            }
        }
        // the bulk stores must have read their shared-memory source before the CTA's shared memory is given up; their
        // global writes are complete when the grid is
        if (TMA_OUT && lane == 0) tma_store_wait_read();
    }
    __syncthreads();
    if constexpr (PAIR) cluster_sync_all();  // the peer no longer reads this CTA's shared memory or signals its barriers
    if (warp == 1) {
        tc_fence_after();
        if constexpr (PAIR) tmem_dealloc_pair(tmem_base, TMEM_COLS);
        else tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ------------------------------------------------------------------------------------------------------ host side
static int64_t dense_ld(int64_t red) { return round_up(red, 8); }  // row stride is a multiple of 16 bytes for TMA

bool tc_dense_supported(const Geo &geo, int dtype) {
    const size_t es = dtype == NMG_F32 ? 4 : 2;
    if (geo.cc > 32767 || geo.C > 65535) return false;
    return expand_smem_bytes(geo, es, false, 1) <= 200 * 1024 && expand_smem_bytes(geo, es, true, 1) <= 200 * 1024;
}

size_t tc_dense_workspace_bytes(const Geo &geo, int dtype, bool transposed) {
    const int64_t rows = transposed ? geo.K : geo.M, red = transposed ? geo.M : geo.K;
    const size_t planes = dtype == NMG_F32 ? 3 : 1;
    return planes * (size_t)rows * (size_t)dense_ld(red) * 2 + 512;
}

template <typename T, bool TR, int N_, bool PLAIN> static int expand_launch_n(const ExpandParams &p, size_t smem, int64_t items, cudaStream_t st) {
    int dev = 0, sms = 148;
    NMG_CUDA(cudaGetDevice(&dev));
    NMG_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const int64_t cap = (int64_t)sms * 16;
    NMG_CUDA(cudaFuncSetAttribute(expand_dense_kernel<T, TR, N_, PLAIN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    expand_dense_kernel<T, TR, N_, PLAIN><<<(unsigned)(items < cap ? items : cap), EXPAND_THREADS, smem, st>>>(p);
    NMG_CUDA(cudaGetLastError());
    return NMG_OK;
}
template <typename T, bool TR, bool PLAIN = false> static int expand_launch(const ExpandParams &p, size_t smem, int64_t items, cudaStream_t st) {
    // the vectorised scatter reads 16-byte pieces of val / idx: tile bases are 16-byte aligned when cc is a multiple of 8
    const bool aligned = (reinterpret_cast<uintptr_t>(p.val) & 15) == 0 && (reinterpret_cast<uintptr_t>(p.idx) & 15) == 0;
    if (aligned && p.n == 1) return expand_launch_n<T, TR, 1, PLAIN>(p, smem, items, st);
    if (aligned && p.n == 2) return expand_launch_n<T, TR, 2, PLAIN>(p, smem, items, st);
    return expand_launch_n<T, TR, 0, PLAIN>(p, smem, items, st);
}

template <typename T, bool PAIR, bool TMA_OUT> static int gemm_launch_as(const GemmParams &p, const GemmMaps &maps, cudaStream_t st) {
    const size_t smem = (size_t)GEMM_RING_BYTES + GEMM_STAGING_BYTES + 256 + 1024;
    int dev = 0, sms = 148;
    NMG_CUDA(cudaGetDevice(&dev));
    NMG_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const int64_t tiles = (int64_t)p.tiles_f * p.tiles_t;
    if (tiles > 0x3fffffff) NMG_FAIL(NMG_ERR_UNSUPPORTED, "too many output tiles for one launch");
    NMG_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<T, PAIR, TMA_OUT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    cudaLaunchConfig_t cfg = {};
    const int64_t units = PAIR ? sms / 2 : sms;  // persistent CTAs, or CTA pairs
    cfg.gridDim = dim3((unsigned)((tiles < units ? tiles : units) * (PAIR ? 2 : 1)));
    cfg.blockDim = dim3(GEMM_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // overlap the prologue with the expansion pass's tail
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = 2;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = PAIR ? 2 : 1;
    NMG_CUDA(cudaLaunchKernelEx(&cfg, gemm_tc_kernel<T, PAIR, TMA_OUT>, p, maps));
    return NMG_OK;
}
template <typename T, bool PAIR> static int gemm_launch(const GemmParams &p, const GemmMaps &maps, cudaStream_t st) {
    return p.out_tma ? gemm_launch_as<T, PAIR, true>(p, maps, st) : gemm_launch_as<T, PAIR, false>(p, maps, st);
}

// CTA pairs serve 16-bit operands when the output has at least two 128-feature tiles (a pair covers 256 features).
bool tc_dense_uses_pair(const Geo &geo, int dtype, bool transposed) {
    return dtype != NMG_F32 && (transposed ? geo.K : geo.M) > TC_BM;
}

// (val, idx) -> the weight with its zeros restored, rows `ld` elements apart at `dst` (16-byte aligned, ld a multiple of 8).
// plain = false: the matmul's operand, 16-bit or three bf16 planes for fp32 (plane_rows rows each); plain = true: the
// weight in its own dtype (the densifier), where full 8-element stores must not run past the row: K a multiple of 8.
static int expand_to(const Geo &geo, int dtype, bool transposed, bool plain, const void *val, const int16_t *idx, void *dst, int64_t ld,
                     cudaStream_t st) {
    const int64_t rows = transposed ? geo.K : geo.M;
    const size_t es = dtype == NMG_F32 ? 4 : 2;
    int rc;
    PatternTable tab;
    if ((rc = get_pattern_table(geo.n, geo.m, &tab))) return rc;
    ExpandParams ep{};
    ep.val = val; ep.idx = idx; ep.order = tab.order; ep.dst = dst;
    ep.ld = ld; ep.plane_elems = rows * ld;
    ep.M = geo.M; ep.K = geo.K; ep.nb = geo.nb; ep.nc = geo.nc;
    ep.n = geo.n; ep.m = geo.m; ep.g = geo.g; ep.C = geo.C; ep.cc = geo.cc;
    ep.R = expand_rows_per_item(geo, es, transposed);
    ep.pitch = expand_pitch(geo, transposed, ep.R);
    const size_t esmem = expand_smem_bytes(geo, es, transposed, ep.R);
    if (esmem > 200 * 1024) NMG_FAIL(NMG_ERR_UNSUPPORTED, "chunk of %d columns does not fit the expansion pass", geo.cc);
    const int64_t items = ((geo.nb + ep.R - 1) / ep.R) * geo.nc;
    if (dtype == NMG_F16) return transposed ? expand_launch<__half, true>(ep, esmem, items, st) : expand_launch<__half, false>(ep, esmem, items, st);
    if (dtype == NMG_BF16) return transposed ? expand_launch<__nv_bfloat16, true>(ep, esmem, items, st) : expand_launch<__nv_bfloat16, false>(ep, esmem, items, st);
    if (plain) return expand_launch<float, false, true>(ep, esmem, items, st);
    return transposed ? expand_launch<float, true>(ep, esmem, items, st) : expand_launch<float, false>(ep, esmem, items, st);
}

int tc_dense_expand(const Geo &geo, int dtype, bool transposed, const void *val, const int16_t *idx, char *dense, cudaStream_t st) {
    return expand_to(geo, dtype, transposed, false, val, idx, dense, dense_ld(transposed ? geo.M : geo.K), st);
}

// The densifier through the expansion pass: whole tiles are scattered into shared memory and leave as 16-byte stores.
bool tc_expand_plain_supported(const Geo &geo, int dtype, const void *dense, int64_t ld) {
    const size_t es = dtype == NMG_F32 ? 4 : 2;
    if (geo.cc > 32767 || geo.C > 65535 || geo.K % 8 != 0 || ld % 8 != 0 || (reinterpret_cast<uintptr_t>(dense) & 15) != 0) return false;
    return expand_smem_bytes(geo, es, false, expand_rows_per_item(geo, es, false)) <= 200 * 1024;
}
int tc_expand_plain(const Geo &geo, int dtype, const void *val, const int16_t *idx, void *dense, int64_t ld, cudaStream_t st) {
    return expand_to(geo, dtype, false, true, val, idx, dense, ld, st);
}

// out = dense[rows][round_up(red, 8)] (16-bit, or three bf16 planes for fp32) x activations.  act_maps: tensor maps of the
// activation planes (128-byte swizzle; box 64 x 128 when `pair`, else 64 x 256), one for 16-bit data, three for the fp32 split.
int tc_dense_gemm(int64_t rows, int64_t red, int dtype, bool pair, const char *dense, const CUtensorMap *act_maps, int64_t tokens,
                  const void *bias, void *const *outs, int n_outs, void *mc_out, int64_t ld_out, int out_token_major, cudaStream_t st,
                  const Epilogue &epi) {
    if (n_outs < 1 || n_outs > GEMM_MAX_OUTS) NMG_FAIL(NMG_ERR_INVALID, "between 1 and %d output buffers, got %d", GEMM_MAX_OUTS, n_outs);
    const int64_t ld = dense_ld(red);
    const int planes = dtype == NMG_F32 ? 3 : 1;
    int rc;
    GemmMaps maps;
    const int edt = dtype == NMG_F32 ? NMG_BF16 : dtype;
    const size_t osz = dtype == NMG_F32 ? 4 : 2;
    // Token-major output of a CTA-pair product: exchange the operands' roles.  Both boxes are 64 x 128 in pair mode, so the
    // activations can be the row operand (tokens on the accumulator's lanes) and the weight the column operand; the
    // output is then "feature-major" in the kernel's terms -- accumulator rows are output rows -- and leaves through the
    // staged 16-byte path with no transposition, the bias running along the columns.
    const bool swap = pair && out_token_major && n_outs == 1 && !mc_out && tokens > TC_BM && (ld_out * osz) % 16 == 0 &&
                      (reinterpret_cast<uintptr_t>(outs[0]) & 15) == 0;
    for (int c = 0; c < 3; c++) {
        const int pc = c < planes ? c : 0;
        CUtensorMap wmap;
        if ((rc = encode_tmap_2d(&wmap, edt, dense + (size_t)pc * rows * ld * 2, (uint64_t)red, (uint64_t)rows, (uint64_t)ld, TC_BK, TC_BM, 1))) return rc;
        maps.a[c] = swap ? act_maps[c] : wmap;
        maps.b[c] = swap ? wmap : act_maps[c];
    }
    if (swap) {  // from here on "rows" are the accumulator's rows (tokens) and "tokens" its columns (output features)
        const int64_t t = rows;
        rows = tokens;
        tokens = t;
        out_token_major = 0;
    }
    int *status = nullptr;
    if ((rc = get_status_word(&status))) return rc;
    GemmParams gp{};
    gp.bias = bias;
    gp.n_out = n_outs;
    gp.bias_cols = swap ? 1 : 0;
    bool vec = !out_token_major && (ld_out * osz) % 16 == 0;
    for (int d = 0; d < n_outs; d++) {
        if (!outs[d]) NMG_FAIL(NMG_ERR_INVALID, "output buffer %d is NULL", d);
        gp.outs[d] = outs[d];
        vec = vec && (reinterpret_cast<uintptr_t>(outs[d]) & 15) == 0;
    }
    gp.out_feats = rows; gp.red = red; gp.ntok = tokens; gp.ld_out = ld_out;
    gp.out_token_major = out_token_major;
    gp.out_staged = vec ? 1 : 0;
    gp.out_tm_vec = (out_token_major && n_outs == 1 && (ld_out * osz) % 16 == 0 && (reinterpret_cast<uintptr_t>(outs[0]) & 15) == 0 &&
                     (!epi.residual || ((epi.ld_res * osz) % 16 == 0 && (reinterpret_cast<uintptr_t>(epi.residual) & 15) == 0)))
                        ? 1 : 0;
    gp.out_tma = (vec && n_outs == 1 && !mc_out) ? 1 : 0;
    if (gp.out_tma) {
        const uint32_t box_cols = (uint32_t)(128 / osz);
        if ((rc = encode_tmap_2d(&maps.out, dtype, outs[0], (uint64_t)tokens, (uint64_t)rows, (uint64_t)ld_out, box_cols, 32, 1))) return rc;
    } else {
        maps.out = maps.a[0];  // never used; keeps the parameter defined
    }
    gp.mc_out = (vec && mc_out && (reinterpret_cast<uintptr_t>(mc_out) & 15) == 0) ? mc_out : nullptr;
    const int tile_feats = pair ? 2 * TC_BM : TC_BM;
    gp.tiles_f = (int)((rows + tile_feats - 1) / tile_feats);
    gp.tiles_t = (int)((tokens + TC_BN - 1) / TC_BN);
    gp.band = pair ? TC_BAND_PAIR : TC_BAND;
    {
        // many waves over a long reduction: keep the producers in step (see the kernel); the counter is zeroed in stream order
        int dev = 0, sms = 148;
        NMG_CUDA(cudaGetDevice(&dev));
        NMG_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        const int64_t units = pair ? sms / 2 : sms;
        if ((int64_t)gp.tiles_f * gp.tiles_t >= 3 * units && red >= 4096) {
            if ((rc = get_wave_counter(&gp.wave_ctr))) return rc;
            NMG_CUDA(cudaMemsetAsync(gp.wave_ctr, 0, sizeof(unsigned), st));
        }
    }
    gp.status = status;
    gp.act = epi.act; gp.residual = epi.residual; gp.ld_res = epi.ld_res;
    gp.res_vec = (epi.residual && (epi.ld_res * osz) % 16 == 0 && (reinterpret_cast<uintptr_t>(epi.residual) & 15) == 0) ? 1 : 0;
    if (dtype == NMG_F32) return gemm_launch<float, false>(gp, maps, st);
    if (dtype == NMG_F16) return pair ? gemm_launch<__half, true>(gp, maps, st) : gemm_launch<__half, false>(gp, maps, st);
    return pair ? gemm_launch<__nv_bfloat16, true>(gp, maps, st) : gemm_launch<__nv_bfloat16, false>(gp, maps, st);
}

// Two passes: expansion into `ws`, then the matmul on the expanded weight.
int tc_dense_matmul(const Geo &geo, int dtype, bool transposed, const void *val, const int16_t *idx, const CUtensorMap *act_maps,
                    int64_t tokens, const void *bias, void *const *outs, int n_outs, void *mc_out, int64_t ld_out, int out_token_major,
                    void *ws, size_t ws_bytes, cudaStream_t st, const Epilogue &epi) {
    const int64_t rows = transposed ? geo.K : geo.M, red = transposed ? geo.M : geo.K;
    const size_t need = tc_dense_workspace_bytes(geo, dtype, transposed);
    if (!ws || ws_bytes < need) NMG_FAIL(NMG_ERR_WORKSPACE, "workspace of %zu bytes required for the expanded weight, got %zu", need, ws_bytes);
    char *dense = reinterpret_cast<char *>(((uintptr_t)ws + 255) & ~(uintptr_t)255);
    int rc;
    if ((rc = tc_dense_expand(geo, dtype, transposed, val, idx, dense, st))) return rc;
    return tc_dense_gemm(rows, red, dtype, tc_dense_uses_pair(geo, dtype, transposed), dense, act_maps, tokens, bias, outs, n_outs, mc_out,
                         ld_out, out_token_major, st, epi);
}

}  // namespace nmg
