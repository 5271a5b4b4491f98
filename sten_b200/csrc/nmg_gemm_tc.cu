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
//                         MMAs (128 x 256 x 16, fp32 accumulators in TMEM), warps 2..5 drain accumulators.  16-bit
//                         mode double-buffers the accumulator (2 x 256 TMEM columns) so that the drain of one tile
//                         overlaps the MMAs of the next; fp32 mode uses the second half for the running sum into which
//                         the tensor core's partial tile is promoted every TC_CHUNK_KB k-blocks.
//
// All device-side waits are bounded: a wait that runs out sets the status word and the role leaves its loop; the
// CTA then meets at the common exit where TMEM is released.
#include <cstdlib>

#include "nmg_spmm_simt.cuh"
#include "nmg_tc_common.cuh"

namespace nmg {

// =========================================================================================================
// Expansion pass
// =========================================================================================================
struct ExpandParams {
    const void *val;            // [tiles][C][g][n]
    const int16_t *idx;         // [tiles][C][g]
    const int8_t *slot_of_row;  // [C][m]: slot that holds row r under pattern p, or -1
    void *dst;                  // [planes][rows][ld] 16-bit
    int64_t ld, plane_elems;
    int64_t M, K, nb, nc;
    int n, m, g, C, cc;
    int R;                      // row-blocks per work item
};

constexpr int EXPAND_THREADS = 256;

__device__ __forceinline__ void split3(float f, __nv_bfloat16 &hi, __nv_bfloat16 &mid, __nv_bfloat16 &lo) {
    hi = __float2bfloat16_rn(f);
    const float r1 = f - __bfloat162float(hi);
    mid = __float2bfloat16_rn(r1);
    lo = __float2bfloat16_rn(r1 - __bfloat162float(mid));
}

// One element (PAIR = false) or two adjacent elements starting at an even offset (PAIR = true).
template <typename T, bool PAIR> __device__ __forceinline__ void expand_store(const ExpandParams &p, int64_t off, T a, T b) {
    if constexpr (sizeof(T) == 2) {
        T *d = static_cast<T *>(p.dst) + off;
        if (PAIR) *reinterpret_cast<uint32_t *>(d) = (uint32_t)bits16<T>(a) | ((uint32_t)bits16<T>(b) << 16);
        else *d = a;
    } else {
        __nv_bfloat16 pa[3], pb[3];
        split3(a, pa[0], pa[1], pa[2]);
        split3(b, pb[0], pb[1], pb[2]);
#pragma unroll
        for (int c = 0; c < 3; c++) {
            __nv_bfloat16 *d = static_cast<__nv_bfloat16 *>(p.dst) + c * p.plane_elems + off;
            if (PAIR) *reinterpret_cast<uint32_t *>(d) = (uint32_t)__bfloat16_as_ushort(pa[c]) | ((uint32_t)__bfloat16_as_ushort(pb[c]) << 16);
            else *d = pa[c];
        }
    }
}

// Work item = (column chunk kc, R consecutive row-blocks).  The item's values and an inverse index (column -> slot,
// pattern) are staged in shared memory; then every output element is looked up and written in the orientation the
// matmul wants, lanes along the contiguous axis of the destination.
template <typename T, bool TR>
__global__ void __launch_bounds__(EXPAND_THREADS) expand_dense_kernel(const ExpandParams prm) {
    extern __shared__ __align__(16) char smem[];
    const int n = prm.n, m = prm.m, g = prm.g, cc = prm.cc, R = prm.R;
    T *sval = reinterpret_cast<T *>(smem);                                                            // [R][cc * n]
    uint32_t *code = reinterpret_cast<uint32_t *>(smem + (((size_t)R * cc * n * sizeof(T) + 15) & ~(size_t)15));  // [R][cc]: pattern << 16 | slot
    int8_t *sor = reinterpret_cast<int8_t *>(code + (size_t)R * cc);                                  // [C][m]
    for (int i = threadIdx.x; i < prm.C * m; i += EXPAND_THREADS) sor[i] = prm.slot_of_row[i];

    const T *val = static_cast<const T *>(prm.val);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int NW = EXPAND_THREADS / 32;
    const int64_t groups = (prm.nb + R - 1) / R;
    const int64_t items = groups * prm.nc;
    const T zero = DT<T>::from_f32(0.f);

    auto value = [&](int j, int r, int c) -> T {
        const uint32_t cd = code[j * cc + c];
        if (cd == 0xffffffffu) return zero;
        const int t = sor[(cd >> 16) * m + r];
        return t >= 0 ? sval[(size_t)j * cc * n + (cd & 0xffffu) * n + t] : zero;
    };

    for (int64_t item = blockIdx.x; item < items; item += gridDim.x) {
        const int64_t kc = item / groups, mb0 = (item - kc * groups) * R;
        const int rj = (int)(prm.nb - mb0 < R ? prm.nb - mb0 : R);  // row-blocks in this item
        __syncthreads();  // previous item fully written out
        for (int e = threadIdx.x; e < rj * cc; e += EXPAND_THREADS) code[e] = 0xffffffffu;
        // tiles of consecutive row-blocks of one chunk are consecutive in memory
        const T *vsrc = val + (kc * prm.nb + mb0) * (int64_t)cc * n;
        for (int e = threadIdx.x; e < rj * cc * n; e += EXPAND_THREADS) sval[e] = vsrc[e];
        __syncthreads();
        const int16_t *isrc = prm.idx + (kc * prm.nb + mb0) * (int64_t)cc;
        for (int e = threadIdx.x; e < rj * cc; e += EXPAND_THREADS) {
            const int c = isrc[e];
            const int j = e / cc, s = e - j * cc;
            if (c >= 0 && c < cc) code[j * cc + c] = ((uint32_t)(s / g) << 16) | (uint32_t)s;  // a malformed index is ignored
        }
        __syncthreads();
        const int64_t col0 = kc * cc;
        const int ncol = (int)(prm.K - col0 < cc ? prm.K - col0 : cc);  // columns of this chunk inside the weight
        if (!TR) {
            // dst[row][col0 + c]: a warp per output row, lanes along columns
            const bool pairs = ((cc & 1) == 0);
            for (int rr = warp; rr < rj * m; rr += NW) {
                const int j = rr / m, r = rr - j * m;
                const int64_t row = (mb0 + j) * m + r;
                if (row >= prm.M) continue;
                const int64_t base = row * prm.ld + col0;
                if (pairs) {
                    for (int c = 2 * lane; c < ncol; c += 64) {
                        if (c + 1 < ncol) expand_store<T, true>(prm, base + c, value(j, r, c), value(j, r, c + 1));
                        else expand_store<T, false>(prm, base + c, value(j, r, c), zero);
                    }
                } else {
                    for (int c = lane; c < ncol; c += 32) expand_store<T, false>(prm, base + c, value(j, r, c), zero);
                }
            }
        } else {
            // dst[col0 + c][mb0 * m + e]: a warp per weight column, lanes along the rj * m weight rows of the item
            const bool pairs = ((m & 1) == 0);
            const int seg = rj * m;
            const int64_t r0 = mb0 * m;
            for (int c = warp; c < ncol; c += NW) {
                const int64_t base = (col0 + c) * prm.ld + r0;
                if (pairs) {
                    for (int e = 2 * lane; e < seg; e += 64) {
                        if (r0 + e >= prm.M) break;
                        const int j = e / m, r = e - j * m;
                        if (r0 + e + 1 < prm.M) expand_store<T, true>(prm, base + e, value(j, r, c), value(j, r + 1, c));
                        else expand_store<T, false>(prm, base + e, value(j, r, c), zero);
                    }
                } else {
                    for (int e = lane; e < seg; e += 32) {
                        if (r0 + e >= prm.M) break;
                        const int j = e / m, r = e - j * m;
                        expand_store<T, false>(prm, base + e, value(j, r, c), zero);
                    }
                }
            }
        }
    }
}

static size_t expand_smem_bytes(const Geo &geo, size_t es, int R) {
    return (((size_t)R * geo.cc * geo.n * es + 15) & ~(size_t)15) + (size_t)R * geo.cc * 4 + (size_t)geo.C * geo.m + 16;
}
static int expand_rows_per_item(const Geo &geo, size_t es) {
    int R = 64 / geo.m;
    if (R < 1) R = 1;
    while (R > 1 && expand_smem_bytes(geo, es, R) > 96 * 1024) R >>= 1;
    return R;
}

// =========================================================================================================
// Dense-operand matmul
// =========================================================================================================
constexpr int GEMM_THREADS = 32 * 6;  // TMA warp, MMA warp, four drain warps (one per TMEM lane quarter)
constexpr int GEMM_STAGE_BYTES = TC_A_BYTES + TC_B_BYTES;

struct GemmParams {
    const void *bias;  // [out_feats] or NULL
    void *out;
    int64_t out_feats, red, ntok, ld_out;
    int out_token_major;
    int tiles_f, tiles_t;
    int *status;
};

struct GemmMaps {
    CUtensorMap a[3];  // weight planes, box 64 x 128, 128-byte swizzle
    CUtensorMap b[3];  // activation planes, box 64 x 256
};

template <typename T>
__global__ void __launch_bounds__(GEMM_THREADS, 1) gemm_tc_kernel(const GemmParams prm, const __grid_constant__ GemmMaps maps) {
    constexpr int TERMS = TcMode<T>::TERMS;
    using E = typename TcMode<T>::elem;
    constexpr bool SPLIT = TERMS > 1;
    constexpr int NBUF = SPLIT ? 1 : 2;  // accumulator tiles in flight between the MMA issuer and the drain warps
    constexpr uint32_t TMEM_COLS = 2 * TC_ACC_COLS;

    extern __shared__ char smem_raw[];
    char *smem = reinterpret_cast<char *>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    char *misc = smem + TC_STAGES * GEMM_STAGE_BYTES;
    uint64_t *full = reinterpret_cast<uint64_t *>(misc);
    uint64_t *empty = full + TC_STAGES;
    uint64_t *acc_full = empty + TC_STAGES;  // [2] MMA issuer -> drain warps: unit complete in accumulator b
    uint64_t *acc_free = acc_full + 2;       // [2] drain warps -> MMA issuer: accumulator b may be overwritten
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(misc + 128);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // A "unit" is what the MMA issuer hands to the drain warps: a whole tile (16-bit) or a chunk of k-blocks (fp32).
    const int ntiles = prm.tiles_f * prm.tiles_t;
    const int my_tiles = ((int)blockIdx.x < ntiles) ? (ntiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
    const int nkb = (int)((prm.red + TC_BK - 1) / TC_BK) * TERMS;  // iterations per tile: k-blocks x split terms (term fastest)
    const int chunk_it = SPLIT ? TC_CHUNK_KB * TERMS : nkb;
    const int nchunks = (nkb + chunk_it - 1) / chunk_it;

    if (tid == 0) {
        for (int s = 0; s < TC_STAGES; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_free[b], 4);  // lane 0 of each drain warp
        }
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    auto tile_origin = [&](int ti, int &feat0, int &tok0) {
        int tile_f, tile_t;
        tile_of_cta((int)blockIdx.x + ti * (int)gridDim.x, prm.tiles_f, prm.tiles_t, tile_f, tile_t);
        feat0 = tile_f * TC_BM;
        tok0 = tile_t * TC_BN;
    };

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (one lane)
        if (lane == 0) {
            int it = 0;
            bool ok = true;
            for (int ti = 0; ti < my_tiles && ok; ti++) {
                int feat0, tok0;
                tile_origin(ti, feat0, tok0);
                for (int kb = 0; kb < nkb; kb++, it++) {
                    const int s = it % TC_STAGES;
                    const uint32_t ph = (uint32_t)((it / TC_STAGES) & 1);
                    if (!(ok = mbar_wait_bounded(&empty[s], ph ^ 1, prm.status, 21))) break;
                    mbar_expect_tx(&full[s], GEMM_STAGE_BYTES);
                    const int term = kb % TERMS;
                    const int wc = TERMS == 1 ? 0 : kSplitW[term], xc = TERMS == 1 ? 0 : kSplitX[term];
                    char *stage = smem + s * GEMM_STAGE_BYTES;
                    tma_load_2d(stage, &maps.a[wc], (kb / TERMS) * TC_BK, feat0, &full[s]);
                    tma_load_2d(stage + TC_A_BYTES, &maps.b[xc], (kb / TERMS) * TC_BK, tok0, &full[s]);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (one lane)
        if (lane == 0) {
            const uint32_t idesc = make_idesc<E>();
            bool ok = true;
            int it = 0, unit = 0;
            for (int ti = 0; ti < my_tiles && ok; ti++) {
                int kb = 0;
                for (int c = 0; c < nchunks && ok; c++, unit++) {
                    const int b = unit % NBUF, use = unit / NBUF;
                    if (use > 0) ok = mbar_wait_bounded(&acc_free[b], (uint32_t)((use - 1) & 1), prm.status, 26);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t d_tmem = tmem_base + (uint32_t)(b * TC_ACC_COLS);
                    const int kend = (kb + chunk_it < nkb) ? kb + chunk_it : nkb;
                    for (bool first = true; kb < kend; kb++, it++, first = false) {
                        const int s = it % TC_STAGES;
                        const uint32_t ph = (uint32_t)((it / TC_STAGES) & 1);
                        if (!(ok = mbar_wait_bounded(&full[s], ph, prm.status, 22))) break;
                        tc_fence_after();
                        const uint64_t adesc = make_sw128_desc(smem_u32(smem + s * GEMM_STAGE_BYTES));
                        const uint64_t bdesc = make_sw128_desc(smem_u32(smem + s * GEMM_STAGE_BYTES + TC_A_BYTES));
#pragma unroll
                        for (int k = 0; k < TC_BK / 16; k++)  // 16 elements = 32 bytes = 2 descriptor units per step
                            tc_mma_f16(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (first && k == 0) ? 0u : 1u);
                        tc_commit(&empty[s]);  // arrives when the MMAs above have read the stage
                    }
                    tc_commit(&acc_full[b]);   // arrives when the unit's MMAs have written TMEM (also on the error path)
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ drain warps: promotion and epilogue
        const int q = warp & 3;  // TMEM lane quarter this warp may access
        const uint32_t lane_base = tmem_base + ((uint32_t)(q * 32) << 16);
        T *out = static_cast<T *>(prm.out);
        int unit = 0;
        bool ok = true;
        for (int ti = 0; ti < my_tiles && ok; ti++) {
            int feat0, tok0;
            tile_origin(ti, feat0, tok0);
            const int64_t feat = (int64_t)feat0 + q * 32 + lane;
            const bool feat_ok = feat < prm.out_feats;
            const float bias = (prm.bias && feat_ok) ? DT<T>::to_f32(static_cast<const T *>(prm.bias)[feat]) : 0.f;
            for (int c = 0; c < nchunks; c++, unit++) {
                const int b = unit % NBUF, use = unit / NBUF;
                if (!(ok = mbar_wait_bounded(&acc_full[b], (uint32_t)(use & 1), prm.status, 25))) break;
                tc_fence_after();
                const bool last = c == nchunks - 1;
                for (int sl = 0; sl < TC_BN / 32; sl++) {
                    uint32_t r[32];
                    tmem_ld32(lane_base + (uint32_t)(b * TC_ACC_COLS + sl * 32), r);
                    if (SPLIT && c > 0) {
                        uint32_t run[32];
                        tmem_ld32(lane_base + (uint32_t)(TC_ACC_COLS + sl * 32), run);
#pragma unroll
                        for (int j = 0; j < 32; j++) r[j] = __float_as_uint(__fadd_rn(__uint_as_float(run[j]), __uint_as_float(r[j])));
                    }
                    if (!last) {
                        tmem_st32(lane_base + (uint32_t)(TC_ACC_COLS + sl * 32), r);
                        continue;
                    }
                    const int64_t tokc = (int64_t)tok0 + sl * 32;
                    if (tokc >= prm.ntok || !feat_ok) continue;
                    const bool vec = !prm.out_token_major && tokc + 32 <= prm.ntok && (prm.ld_out % (16 / (int)sizeof(T))) == 0 &&
                                     (reinterpret_cast<uintptr_t>(out) & 15) == 0;
                    if (vec) {  // 32 consecutive tokens of this feature: 16-byte stores
                        uint4 *dst = reinterpret_cast<uint4 *>(out + feat * prm.ld_out + tokc);
                        if constexpr (sizeof(T) == 4) {
#pragma unroll
                            for (int v = 0; v < 8; v++)
                                dst[v] = make_uint4(__float_as_uint(__uint_as_float(r[4 * v]) + bias), __float_as_uint(__uint_as_float(r[4 * v + 1]) + bias),
                                                    __float_as_uint(__uint_as_float(r[4 * v + 2]) + bias), __float_as_uint(__uint_as_float(r[4 * v + 3]) + bias));
                        } else {
#pragma unroll
                            for (int v = 0; v < 4; v++) {
                                uint32_t w[4];
#pragma unroll
                                for (int h = 0; h < 4; h++) {
                                    const T lo = DT<T>::from_f32(__uint_as_float(r[8 * v + 2 * h]) + bias);
                                    const T hi = DT<T>::from_f32(__uint_as_float(r[8 * v + 2 * h + 1]) + bias);
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
                                const T o = DT<T>::from_f32(__uint_as_float(r[j]) + bias);
                                if (prm.out_token_major) out[tok * prm.ld_out + feat] = o;
                                else out[feat * prm.ld_out + tok] = o;
                            }
                        }
                    }
                }
                tc_fence_before();  // this warp's TMEM reads of the unit are complete (tcgen05.wait::ld in tmem_ld32)
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_free[b]);
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
static int64_t dense_ld(int64_t red) { return round_up(red, 8); }  // row stride is a multiple of 16 bytes for TMA

bool tc_dense_supported(const Geo &geo, int dtype) {
    const size_t es = dtype == NMG_F32 ? 4 : 2;
    if (geo.cc > 32767 || geo.C > 65535) return false;
    return expand_smem_bytes(geo, es, 1) <= 200 * 1024;
}

size_t tc_dense_workspace_bytes(const Geo &geo, int dtype, bool transposed) {
    const int64_t rows = transposed ? geo.K : geo.M, red = transposed ? geo.M : geo.K;
    const size_t planes = dtype == NMG_F32 ? 3 : 1;
    return planes * (size_t)rows * (size_t)dense_ld(red) * 2 + 512;
}

template <typename T, bool TR> static int expand_launch(const ExpandParams &p, size_t smem, int64_t items, cudaStream_t st) {
    int dev = 0, sms = 148;
    NMG_CUDA(cudaGetDevice(&dev));
    NMG_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const int64_t cap = (int64_t)sms * 16;
    NMG_CUDA(cudaFuncSetAttribute(expand_dense_kernel<T, TR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    expand_dense_kernel<T, TR><<<(unsigned)(items < cap ? items : cap), EXPAND_THREADS, smem, st>>>(p);
    NMG_CUDA(cudaGetLastError());
    return NMG_OK;
}

template <typename T> static int gemm_launch(const GemmParams &p, const GemmMaps &maps, cudaStream_t st) {
    const size_t smem = (size_t)TC_STAGES * GEMM_STAGE_BYTES + 256 + 1024;
    int dev = 0, sms = 148;
    NMG_CUDA(cudaGetDevice(&dev));
    NMG_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const int64_t tiles = (int64_t)p.tiles_f * p.tiles_t;
    if (tiles > 0x3fffffff) NMG_FAIL(NMG_ERR_UNSUPPORTED, "too many output tiles for one launch");
    NMG_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    gemm_tc_kernel<T><<<(unsigned)(tiles < sms ? tiles : sms), GEMM_THREADS, smem, st>>>(p, maps);  // persistent
    NMG_CUDA(cudaGetLastError());
    return NMG_OK;
}

// act_maps: tensor maps of the activation planes (box 64 x 256, 128-byte swizzle), one for 16-bit data, three for
// the fp32 split.  ws holds the expanded weight for the duration of the call.
int tc_dense_matmul(const Geo &geo, int dtype, bool transposed, const void *val, const int16_t *idx, const CUtensorMap *act_maps,
                    int64_t tokens, const void *bias, void *out, int64_t ld_out, int out_token_major, void *ws, size_t ws_bytes,
                    cudaStream_t st) {
    const int64_t rows = transposed ? geo.K : geo.M, red = transposed ? geo.M : geo.K;
    const size_t need = tc_dense_workspace_bytes(geo, dtype, transposed);
    if (!ws || ws_bytes < need) NMG_FAIL(NMG_ERR_WORKSPACE, "workspace of %zu bytes required for the expanded weight, got %zu", need, ws_bytes);
    char *dense = reinterpret_cast<char *>(((uintptr_t)ws + 255) & ~(uintptr_t)255);
    const int64_t ld = dense_ld(red);
    const int planes = dtype == NMG_F32 ? 3 : 1;
    const size_t es = dtype == NMG_F32 ? 4 : 2;
    int rc;
    PatternTable tab;
    if ((rc = get_pattern_table(geo.n, geo.m, &tab))) return rc;

    ExpandParams ep{};
    ep.val = val; ep.idx = idx; ep.slot_of_row = tab.slot_of_row; ep.dst = dense;
    ep.ld = ld; ep.plane_elems = rows * ld;
    ep.M = geo.M; ep.K = geo.K; ep.nb = geo.nb; ep.nc = geo.nc;
    ep.n = geo.n; ep.m = geo.m; ep.g = geo.g; ep.C = geo.C; ep.cc = geo.cc;
    ep.R = expand_rows_per_item(geo, es);
    const size_t esmem = expand_smem_bytes(geo, es, ep.R);
    if (esmem > 200 * 1024) NMG_FAIL(NMG_ERR_UNSUPPORTED, "chunk of %d columns does not fit the expansion pass", geo.cc);
    const int64_t items = ((geo.nb + ep.R - 1) / ep.R) * geo.nc;
    if (dtype == NMG_F16) rc = transposed ? expand_launch<__half, true>(ep, esmem, items, st) : expand_launch<__half, false>(ep, esmem, items, st);
    else if (dtype == NMG_BF16) rc = transposed ? expand_launch<__nv_bfloat16, true>(ep, esmem, items, st) : expand_launch<__nv_bfloat16, false>(ep, esmem, items, st);
    else rc = transposed ? expand_launch<float, true>(ep, esmem, items, st) : expand_launch<float, false>(ep, esmem, items, st);
    if (rc) return rc;

    GemmMaps maps;
    const int edt = dtype == NMG_F32 ? NMG_BF16 : dtype;
    for (int c = 0; c < 3; c++) {
        const int pc = c < planes ? c : 0;
        if ((rc = encode_tmap_2d(&maps.a[c], edt, dense + (size_t)pc * ep.plane_elems * 2, (uint64_t)red, (uint64_t)rows, (uint64_t)ld, TC_BK, TC_BM, 1))) return rc;
        maps.b[c] = act_maps[c];
    }
    int *status = nullptr;
    if ((rc = get_status_word(&status))) return rc;
    GemmParams gp{bias, out, rows, red, tokens, ld_out, out_token_major, (int)((rows + TC_BM - 1) / TC_BM), (int)((tokens + TC_BN - 1) / TC_BN), status};
    if (dtype == NMG_F16) return gemm_launch<__half>(gp, maps, st);
    if (dtype == NMG_BF16) return gemm_launch<__nv_bfloat16>(gp, maps, st);
    return gemm_launch<float>(gp, maps, st);
}

}  // namespace nmg
