// Transposed product dX = dY W on the structured-sparse tensor cores (tcgen05.mma.sp).
//
// In the format's orientation the n:m blocks run along the weight's ROWS.  In the transposed product
// dX[t][k] = sum_r dY[t][r] W[r][k] the rows r are the reduction axis, so W^T -- the operand whose rows are the output
// features k -- is sparse along the reduction: every aligned group of four rows holds at most two non-zeros whenever
// m is a multiple of 4 and n <= 2 (1:4, 2:4 directly; 1:8, 2:8, 1:16 because a group of four is part of one block).
// That is exactly the 2:4 structure tcgen05.mma.sp multiplies at twice the dense rate: the A operand carries two
// stored values per group of four plus two 2-bit positions, the zeros are never multiplied.
//
// Two kernels:
//   expand_sp_kernel   (val, idx) -> A_sp[K][R/2] (the kept values of W^T, two per group of four rows, 16-bit) and the
//                      metadata, laid out in 2 KB atoms of 128 features x 128 reduction elements in the order the
//                      tensor core's metadata copy (tcgen05.cp 128x128b) expects.  R = M rounded up to 128.
//   gemm_sp_kernel     persistent CTA pairs (cluster of 2), 256 features x 256 tokens per pair and tile.  Warp 0 of each
//                      CTA issues its TMA loads into a ring of four stages of 128 reduction elements: the A_sp tile of
//                      its 128 features (128 x 64 stored values), their metadata atom, and its half of the dY tile (128
//                      tokens, two boxes of 64 reduction elements).  Warp 1 of the even CTA copies each metadata atom into
//                      TMEM and issues tcgen05.mma.sp.cta_group::2 (256 x 256 x 32 per instruction, fp32 accumulators
//                      in both CTAs' TMEM).  Warps 2..9 drain: each reads its share of the finished accumulator into
//                      registers at once and hands the accumulator back before converting and storing, so the next
//                      tile's MMAs overlap the stores with a single accumulator (the metadata needs TMEM columns too).
//
// All device-side waits are bounded; a wait that runs out sets the status word and the CTA meets at the common exit.
#include "nmg_expand.cuh"
#include "nmg_spmm_simt.cuh"
#include "nmg_tc_common.cuh"

namespace nmg {

constexpr int SP_ATOM = 128;          // features and reduction elements covered by one metadata atom
constexpr int SP_ATOM_BYTES = 2048;   // 128 x 128 elements, 4 bits per group of four
constexpr int SP_ROWS_ITEM = 64;      // weight rows per expansion work item

// =========================================================================================================
// Expansion pass
// =========================================================================================================
struct SpExpandParams {
    ExpandParams base;   // dst unused
    void *asp;           // [K][ld_a] 16-bit: stored values of W^T
    uint8_t *meta;       // [ceil(K / 128)][n_rt] atoms of 2048 bytes
    int64_t ld_a;        // = R / 2
    int64_t n_rt;        // = R / 128
};

// Two stored values and the 4-bit metadata of one group of four consecutive reduction elements (16-bit patterns b[0..4)).
// Metadata = position of the first stored value | position of the second << 2, positions ascending.  Groups with fewer
// than two non-zeros are completed with a zero value at a free position so that the pair stays ascending.
__device__ __forceinline__ uint32_t compress4(const uint16_t *b, uint32_t &nibble) {
    int i0 = -1, i1 = -1;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const bool nz = (b[i] & 0x7fffu) != 0;
        if (nz && i0 < 0) i0 = i;
        else if (nz && i1 < 0) i1 = i;
    }
    uint32_t v0 = 0, v1 = 0;
    if (i0 < 0) { i0 = 0; i1 = 3; }                                     // empty group
    else if (i1 < 0) {
        if (i0 == 3) { v1 = b[3]; i0 = 0; i1 = 3; }                      // single value in the last position: (zero, value)
        else { v0 = b[i0]; i1 = 3; }                                     // (value, zero at position 3)
    } else { v0 = b[i0]; v1 = b[i1]; }
    nibble = (uint32_t)i0 | ((uint32_t)i1 << 2);
    return v0 | (v1 << 16);
}

// Work item = (column chunk kc, 64 consecutive weight rows).  The item's W^T tile (lines = weight columns, 64 rows long)
// is scattered into shared memory as in the dense expansion; every thread then turns 16 consecutive rows of one line
// into 8 stored values (one 16-byte store) and one 16-bit metadata word.
template <typename T, int N_>
__global__ void __launch_bounds__(EXPAND_THREADS) expand_sp_kernel(const SpExpandParams sp) {
    extern __shared__ __align__(16) char smem[];
    const ExpandParams &prm = sp.base;
    const int m = prm.m, cc = prm.cc, R = prm.R, pitch = prm.pitch;
    T *tile = reinterpret_cast<T *>(smem);                                // [cc][pitch]
    int8_t *ord = reinterpret_cast<int8_t *>(tile + (size_t)cc * pitch);  // [C][n]
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");       // the matmul kernel's prologue may overlap this grid
    const int n = N_ > 0 ? N_ : prm.n;
    for (int i = threadIdx.x; i < prm.C * n; i += EXPAND_THREADS) ord[i] = prm.order[i];
    for (int i = threadIdx.x; i < cc * pitch; i += EXPAND_THREADS) tile[i] = DT<T>::from_f32(0.f);

    const int64_t groups = sp.n_rt * (SP_ATOM / SP_ROWS_ITEM);  // row groups of 64 up to the padded reduction length
    const int64_t items = groups * prm.nc;
    uint16_t *asp = static_cast<uint16_t *>(sp.asp);

    for (int64_t item = blockIdx.x; item < items; item += gridDim.x) {
        const int64_t kc = item / groups, grp = item - kc * groups, mb0 = grp * R;
        int64_t left = prm.nb - mb0;
        const int rj = (int)(left < 0 ? 0 : (left < R ? left : R));  // row-blocks that exist (0 in the reduction padding)
        __syncthreads();  // the tile is all zeros again
        if (rj > 0) expand_scatter_item<T, true, N_>(prm, tile, ord, kc, mb0, rj);
        __syncthreads();
        const int64_t col0 = kc * cc, r0 = grp * SP_ROWS_ITEM;
        const int64_t cols = prm.K - col0 < cc ? prm.K - col0 : cc;  // lines inside the weight
        for (int v = threadIdx.x; v < (int)cols * 4; v += EXPAND_THREADS) {
            const int l = v >> 2, s = v & 3;
            uint4 *src = reinterpret_cast<uint4 *>(tile + l * pitch + 16 * s);
            uint4 in[2] = {src[0], src[1]};
            src[0] = make_uint4(0, 0, 0, 0);
            src[1] = make_uint4(0, 0, 0, 0);
            const uint16_t *b = reinterpret_cast<const uint16_t *>(in);
            uint32_t w[4], meta = 0;
#pragma unroll
            for (int q = 0; q < 4; q++) {
                uint32_t nib;
                w[q] = compress4(b + 4 * q, nib);
                meta |= nib << (4 * q);
            }
            const int64_t f = col0 + l, r = r0 + 16 * s;
            *reinterpret_cast<uint4 *>(asp + f * sp.ld_a + (r >> 1)) = make_uint4(w[0], w[1], w[2], w[3]);
            // metadata atom (f / 128, r / 128); inside it, feature fi and the 16-element span s16 of the reduction axis
            const int fi = (int)(f & 127), s16 = (int)((r & 127) >> 4);
            uint8_t *atom = sp.meta + ((f >> 7) * sp.n_rt + (r >> 7)) * SP_ATOM_BYTES;
            const int off = (fi & 7) * 16 + ((fi >> 3) & 1) * 2 + (fi >> 4) * 256 + (s16 & 1) * 128 + (s16 >> 1) * 4;
            *reinterpret_cast<uint16_t *>(atom + off) = (uint16_t)meta;
        }
        // lines outside the weight (last chunk) were never written by valid slots, the tile stays clean
    }
}

// =========================================================================================================
// Matmul: CTA pairs (thread-block cluster of 2, tcgen05 cta_group::2), one 256-feature x 256-token tile per pair.
//
// An SM takes in about 64 bytes per clock from L2.  With one CTA per 128 x 256 tile the operands of 128 reduction
// elements are 18 KB of A_sp + 64 KB of dY per 512 tensor-core clocks, 160 bytes per clock: the tensor core would idle
// most of the time.  Two CTAs on neighbouring SMs therefore share one tile of 256 features: each loads the A_sp rows of
// its own 128 features and only HALF of the dY tile (128 tokens); the MMA (M = 256, issued by the even CTA) reads both
// halves of dY from both shared memories.  Per SM that is 50 KB per 512 clocks.  No load is multicast.
//
// Barrier topology.  full[s] lives in the even ("leader") CTA: both CTAs' TMA loads name the leader's barrier,
// the leader's producer posts the expected bytes of both.  empty[s] / acc_full exist in both CTAs and are
// signalled by multicast tcgen05.commit.  acc_free lives in the leader and collects the drain warps of both CTAs.
// Every wait is bounded and every thread reaches the closing cluster barrier, also after a failed wait.
// =========================================================================================================
constexpr int SP_STAGES = 4;                               // ring of stages, 128 reduction elements each
constexpr int SP_B_HALF = 128 * TC_BK * 2;                 // 16 KB: 128 tokens x 64 reduction elements of dY
constexpr int SP_OFF_B = TC_A_BYTES;                       // stage layout: A_sp tile (16 KB) | two dY boxes (2 x 16 KB) | metadata atom (2 KB)
constexpr int SP_OFF_E = SP_OFF_B + 2 * SP_B_HALF;
constexpr int SP_STAGE = SP_OFF_E + SP_ATOM_BYTES;         // 50 KB
constexpr int SP_PAIR_FEATS = 256;
constexpr int SP_DRAIN_WARPS = 8;
constexpr int SP_THREADS = 32 * (2 + SP_DRAIN_WARPS);
constexpr uint32_t SP_TMEM_COLS = 512;
constexpr uint32_t SP_E_COL = 256;                         // metadata columns: two sets of four, used alternately

constexpr int SP_STAGING_BYTES = SP_DRAIN_WARPS * 2048;  // per drain warp: 32 tokens x 32 features, 16-bit

struct SpGemmParams {
    void *out;            // [tokens][ld_out]
    int out_vec;          // output rows are 16-byte aligned: transposed in shared memory, one tiled bulk store per slice
    int64_t out_feats, red, ntok, ld_out, n_rt;
    int tiles_f, tiles_t; // tiles_f counts 256-feature tiles
    int band;             // width of the tile order's bands, in feature tiles
    unsigned *wave_ctr;   // zeroed counter for the producers' soft rendezvous before every tile, or NULL
    int *status;
};
struct SpGemmMaps {
    CUtensorMap a;  // A_sp [K][R/2], box 64 x 128, 128-byte swizzle
    CUtensorMap b;  // dY [tokens][M], box 64 x 128
    CUtensorMap out;  // dX [tokens][K], box 32 features x 32 tokens, no swizzle (out_vec)
    CUtensorMap e;  // metadata as [atoms * 2][256] 32-bit words, box 256 x 2 = one 2 KB atom
};

// Copy 128 rows x 16 bytes of shared memory (row i at byte i * 16: eight-row groups 128 bytes apart, no swizzle) into
// four TMEM columns of all 128 lanes, in both CTAs of the pair (each from its own shared memory, same offset).
// Descriptor: start address >> 4, leading byte offset (unused: one 16-byte column), stride byte offset 128 >> 4 between
// eight-row groups, version 1, no swizzle.
__device__ __forceinline__ void tc2_copy_meta(uint32_t taddr, uint32_t smem_addr) {
    const uint64_t desc = (uint64_t)((smem_addr >> 4) & 0x3FFF) | ((uint64_t)(128 >> 4) << 16) | ((uint64_t)(128 >> 4) << 32) | ((uint64_t)1 << 46);
    asm volatile("tcgen05.cp.cta_group::2.128x128b [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}
__device__ __forceinline__ void tc2_mma_sp_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t e_tmem, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "tcgen05.mma.sp.cta_group::2.kind::f16 [%0], %1, %2, [%3], %4, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(e_tmem), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Instruction descriptor of the pair: M = 256 across both CTAs, N = 256, A structured-sparse (bit 2); bits 0-1 select the
// metadata column inside an aligned pair of TMEM columns.
template <typename T> __device__ __forceinline__ uint32_t make_idesc_sp_pair() {
    const uint32_t fmt = DT<T>::id == NMG_BF16 ? 1u : 0u;
    return (1u << 2) | (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
}

template <typename T>
__global__ void __launch_bounds__(SP_THREADS, 1) gemm_sp_kernel(const SpGemmParams prm, const __grid_constant__ SpGemmMaps maps) {
    extern __shared__ char smem_raw[];
    char *smem = reinterpret_cast<char *>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    char *staging = smem + SP_STAGES * SP_STAGE;
    char *misc = staging + SP_STAGING_BYTES;
    uint64_t *full = reinterpret_cast<uint64_t *>(misc);     // meaningful in the leader only
    uint64_t *empty = full + SP_STAGES;
    uint64_t *acc_full = empty + SP_STAGES;
    uint64_t *acc_free = acc_full + 1;                        // leader only
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(misc + 248);
    static_assert((2 * SP_STAGES + 2) * 8 <= 248 && SP_STAGE % 1024 == 0, "shared-memory plan");

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const int pair = (int)(blockIdx.x >> 1), npairs = (int)(gridDim.x >> 1);
    const int ntiles = prm.tiles_f * prm.tiles_t;
    const int my_tiles = (pair < ntiles) ? (ntiles - pair + npairs - 1) / npairs : 0;
    const int nst = (int)((prm.red + SP_ATOM - 1) / SP_ATOM);  // stages (128 reduction elements) per output tile

    if (tid == 0) {
        for (int s = 0; s < SP_STAGES; s++) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        mbar_init(acc_full, 1);
        mbar_init(acc_free, 2 * SP_DRAIN_WARPS);  // the drain warps of both CTAs
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc_pair(tmem_slot, SP_TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // barriers of both CTAs are initialised before anyone arrives remotely
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t full_leader = map_to_rank(smem_u32(&full[0]), 0);
    const uint32_t acc_free_leader = map_to_rank(smem_u32(acc_free), 0);

    auto tile_origin = [&](int ti, int &tile_f, int &tok0) {
        int tile_t;
        tile_of_cta(pair + ti * npairs, prm.tiles_f, prm.tiles_t, tile_f, tile_t, prm.band);
        tok0 = tile_t * TC_BN;
    };

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (one lane per CTA)
        if (lane == 0) {
            int it = 0;
            bool ok = true;
            asm volatile("griddepcontrol.wait;" ::: "memory");  // the expansion pass's output arrives through the loads below
            unsigned arrivals = 0;
            for (int ti = 0; ti < my_tiles && ok; ti++) {
                int tile_f, tok0;
                tile_origin(ti, tile_f, tok0);
                const int half_f = tile_f * 2 + (int)rank;  // this CTA's 128-feature tile = its metadata atom row
                if (prm.wave_ctr && ti > 0) {  // keep the CTAs that share operand panels through L2 in step (soft_rendezvous)
                    const int left = ntiles - ti * npairs;
                    arrivals += (unsigned)((left < npairs ? left : npairs) * 2);
                    soft_rendezvous(prm.wave_ctr, arrivals, (uint64_t)nst * 80);
                }
                for (int j = 0; j < nst; j++, it++) {
                    const int s = it % SP_STAGES;
                    if (!(ok = mbar_wait_cluster_bounded(&empty[s], (uint32_t)(((it / SP_STAGES) & 1) ^ 1), prm.status, 31))) break;
                    if (leader) mbar_expect_tx(&full[s], 2 * SP_STAGE);  // both CTAs report to this barrier
                    char *stage = smem + s * SP_STAGE;
                    const uint32_t bar = full_leader + s * 8;
                    tma_load_2d_pair(stage, &maps.a, j * 64, half_f * TC_BM, bar);
                    tma_load_2d_pair(stage + SP_OFF_B, &maps.b, j * SP_ATOM, tok0 + (int)rank * 128, bar);
                    tma_load_2d_pair(stage + SP_OFF_B + SP_B_HALF, &maps.b, j * SP_ATOM + TC_BK, tok0 + (int)rank * 128, bar);
                    tma_load_2d_pair(stage + SP_OFF_E, &maps.e, 0, (int)(((int64_t)half_f * prm.n_rt + j) * 2), bar);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (one lane of the leader)
        if (leader && lane == 0) {
            const uint32_t idesc = make_idesc_sp_pair<T>();
            bool ok = true;
            int it = 0;
            for (int ti = 0; ti < my_tiles && ok; ti++) {
                if (ti > 0) ok = mbar_wait_cluster_bounded(acc_free, (uint32_t)((ti - 1) & 1), prm.status, 36);
                if (!ok) break;
                tc_fence_after();
                for (int j = 0; j < nst; j++, it++) {
                    const int s = it % SP_STAGES;
                    if (!(ok = mbar_wait_cluster_bounded(&full[s], (uint32_t)((it / SP_STAGES) & 1), prm.status, 33))) break;
                    tc_fence_after();
                    const uint32_t stage = smem_u32(smem + s * SP_STAGE);
                    const uint32_t e_set = tmem_base + SP_E_COL + 4u * (uint32_t)(it & 1);
                    tc2_copy_meta(e_set, stage + SP_OFF_E);
                    const uint64_t adesc = make_sw128_desc(stage);
                    const uint64_t bdesc0 = make_sw128_desc(stage + SP_OFF_B), bdesc1 = make_sw128_desc(stage + SP_OFF_B + SP_B_HALF);
#pragma unroll
                    for (int k = 0; k < 4; k++)  // 32 reduction elements per instruction: 16 stored values of A (2 descriptor units), 32 of dY (4 units)
                        tc2_mma_sp_f16(tmem_base, adesc + 2 * k, (k < 2 ? bdesc0 : bdesc1) + 4 * (k & 1), e_set + (uint32_t)(k & 2),
                                       idesc | (uint32_t)(k & 1), (j == 0 && k == 0) ? 0u : 1u);  // metadata columns are addressed in pairs
                    tc2_commit_both(&empty[s]);
                }
                tc2_commit_both(acc_full);  // arrives in both CTAs when the tile's MMAs have written TMEM (also on the error path)
            }
        }
    } else {
        // ------------------------------------------------------------------ drain warps (both CTAs, own 128 features)
        const int q = warp & 3;                                          // TMEM lane quarter this warp may access
        constexpr int SLICES = (TC_BN / 32) / (SP_DRAIN_WARPS / 4);      // 32-column slices per warp: 4
        const int sl0 = ((warp - 2) >> 2) * SLICES;
        const uint32_t lane_base = tmem_base + ((uint32_t)(q * 32) << 16);
        T *out = static_cast<T *>(prm.out);
        bool ok = true;
        for (int ti = 0; ti < my_tiles && ok; ti++) {
            int tile_f, tok0;
            tile_origin(ti, tile_f, tok0);
            const int64_t feat = (int64_t)tile_f * SP_PAIR_FEATS + (int64_t)rank * TC_BM + q * 32 + lane;
            if (!(ok = mbar_wait_cluster_bounded(acc_full, (uint32_t)(ti & 1), prm.status, 35))) break;
            tc_fence_after();
            // the warp's whole share of the accumulator goes to registers first, then the accumulator is handed back:
            // the next tile's MMAs run while this one is converted and stored
            uint32_t r[SLICES][32];
#pragma unroll
            for (int s = 0; s < SLICES; s++) tmem_ld32_issue(lane_base + (uint32_t)((sl0 + s) * 32), r[s]);
#pragma unroll
            for (int s = 0; s < SLICES; s++) tmem_ld_fence(r[s]);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_remote(acc_free_leader);
            if (prm.out_vec) {
                // TMEM hands every lane one feature and 32 tokens per slice; the token-major output wants neighbouring
                // lanes on neighbouring features.  The slice is transposed into a [32 tokens][32 features] tile in shared
                // memory and leaves as one tiled bulk store, clipped by the copy engine at the tensor's edges.
                char *stage_w = staging + (warp - 2) * 2048;
                T *st = reinterpret_cast<T *>(stage_w);
                const int f0 = tile_f * SP_PAIR_FEATS + (int)rank * TC_BM + q * 32;
#pragma unroll
                for (int s = 0; s < SLICES; s++) {
                    const int tokc = tok0 + (sl0 + s) * 32;
                    if (tokc >= prm.ntok) break;  // warp-uniform
                    if (lane == 0) tma_store_wait_read();  // the previous store has read the tile
                    __syncwarp();
#pragma unroll
                    for (int j = 0; j < 32; j++) st[j * 32 + lane] = DT<T>::from_f32(__uint_as_float(r[s][j]));
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0 && f0 < prm.out_feats) tma_store_2d(&maps.out, stage_w, f0, tokc);
                }
                continue;
            }
            if (feat >= prm.out_feats) continue;
#pragma unroll
            for (int s = 0; s < SLICES; s++) {
                const int64_t tokc = (int64_t)tok0 + (sl0 + s) * 32;
                if (tokc >= prm.ntok) break;
                T *p = out + tokc * prm.ld_out + feat;
                if (tokc + 32 <= prm.ntok) {
#pragma unroll
                    for (int j = 0; j < 32; j++, p += prm.ld_out) *p = DT<T>::from_f32(__uint_as_float(r[s][j]));
                } else {
#pragma unroll
                    for (int j = 0; j < 32; j++, p += prm.ld_out)
                        if (tokc + j < prm.ntok) *p = DT<T>::from_f32(__uint_as_float(r[s][j]));
                }
            }
        }
    }
    if (warp >= 2 && lane == 0) tma_store_wait_read();  // sources read before shared memory is given up; writes complete with the grid
    __syncthreads();
    cluster_sync_all();  // the peer no longer reads this CTA's shared memory or signals its barriers
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, SP_TMEM_COLS);
    }
}

// ------------------------------------------------------------------------------------------------------ host side
static int64_t sp_red_padded(const Geo &geo) { return round_up(geo.M, SP_ATOM); }
static int sp_pitch() { return SP_ROWS_ITEM + 8; }
static size_t sp_expand_smem(const Geo &geo) { return (size_t)geo.cc * sp_pitch() * 2 + (size_t)geo.C * geo.n + 16; }

// The structured-sparse path serves 16-bit weights whose blocks are made of whole groups of four rows with at most two
// kept values each: m in {4, 8, 16, 32, 64} (64 % m == 0 keeps expansion items on block boundaries) and n <= 2.
bool tc_sp_supported(const Geo &geo, int dtype) {
    if (dtype != NMG_F16 && dtype != NMG_BF16) return false;
    if (geo.n < 1 || geo.n > 2 || geo.m < 4 || SP_ROWS_ITEM % geo.m != 0) return false;
    return sp_expand_smem(geo) <= 200 * 1024;
}

struct SpLayout { size_t asp_bytes, meta_bytes, total; int64_t ld_a, n_rt, n_ft; };
static SpLayout sp_layout(const Geo &geo) {
    SpLayout l;
    const int64_t R = sp_red_padded(geo);
    l.ld_a = R / 2;
    l.n_rt = R / SP_ATOM;
    l.n_ft = round_up((geo.K + SP_ATOM - 1) / SP_ATOM, 2);  // a CTA pair covers two feature tiles; the second may lie outside the weight
    l.asp_bytes = ((size_t)geo.K * (size_t)l.ld_a * 2 + 255) & ~(size_t)255;
    l.meta_bytes = (size_t)l.n_ft * (size_t)l.n_rt * SP_ATOM_BYTES;
    l.total = l.asp_bytes + l.meta_bytes + 256;
    return l;
}

template <typename T, int N_> static int sp_expand_launch(const SpExpandParams &p, size_t smem, int64_t items, cudaStream_t st) {
    int dev = 0, sms = 148;
    NMG_CUDA(cudaGetDevice(&dev));
    NMG_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const int64_t cap = (int64_t)sms * 16;
    NMG_CUDA(cudaFuncSetAttribute(expand_sp_kernel<T, N_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    expand_sp_kernel<T, N_><<<(unsigned)(items < cap ? items : cap), EXPAND_THREADS, smem, st>>>(p);
    NMG_CUDA(cudaGetLastError());
    return NMG_OK;
}

template <typename T> static int sp_gemm_launch(const SpGemmParams &p, const SpGemmMaps &maps, cudaStream_t st) {
    const size_t smem = (size_t)SP_STAGES * SP_STAGE + SP_STAGING_BYTES + 256 + 1024;
    int dev = 0, sms = 148;
    NMG_CUDA(cudaGetDevice(&dev));
    NMG_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const int64_t tiles = (int64_t)p.tiles_f * p.tiles_t;
    if (tiles > 0x3fffffff) NMG_FAIL(NMG_ERR_UNSUPPORTED, "too many output tiles for one launch");
    NMG_CUDA(cudaFuncSetAttribute(gemm_sp_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    cudaLaunchConfig_t cfg = {};
    const int64_t pairs = sms / 2;
    cfg.gridDim = dim3((unsigned)(2 * (tiles < pairs ? tiles : pairs)));  // persistent CTA pairs
    cfg.blockDim = dim3(SP_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // overlap the prologue with the expansion pass's tail
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    NMG_CUDA(cudaLaunchKernelEx(&cfg, gemm_sp_kernel<T>, p, maps));
    return NMG_OK;
}

// (val, idx) -> compressed transposed copy at `buf` (tc_sp_copy_bytes(geo) bytes, 256-byte aligned): A_sp followed by
// the metadata atoms.  One memset (metadata nibbles start as the valid pair (0, 3): atoms of a ragged last feature tile
// are only partly written) and one kernel.
int tc_sp_pack(const Geo &geo, int dtype, const void *val, const int16_t *idx, void *buf, size_t buf_bytes, cudaStream_t st) {
    if (!tc_sp_supported(geo, dtype)) NMG_FAIL(NMG_ERR_UNSUPPORTED, "the structured-sparse path needs a 16-bit weight with n <= 2 and m in {4, 8, 16, 32, 64}");
    const SpLayout lay = sp_layout(geo);
    if (!buf || buf_bytes < lay.total) NMG_FAIL(NMG_ERR_WORKSPACE, "buffer of %zu bytes required for the compressed transposed weight, got %zu", lay.total, buf_bytes);
    if (reinterpret_cast<uintptr_t>(buf) & 255) NMG_FAIL(NMG_ERR_INVALID, "the compressed transposed copy must be 256-byte aligned");
    char *base = static_cast<char *>(buf);
    char *meta = base + lay.asp_bytes;
    int rc;
    PatternTable tab;
    if ((rc = get_pattern_table(geo.n, geo.m, &tab))) return rc;
    NMG_CUDA(cudaMemsetAsync(meta, 0xCC, lay.meta_bytes, st));

    SpExpandParams sp{};
    ExpandParams &ep = sp.base;
    ep.val = val; ep.idx = idx; ep.order = tab.order; ep.dst = nullptr;
    ep.M = geo.M; ep.K = geo.K; ep.nb = geo.nb; ep.nc = geo.nc;
    ep.n = geo.n; ep.m = geo.m; ep.g = geo.g; ep.C = geo.C; ep.cc = geo.cc;
    ep.R = SP_ROWS_ITEM / geo.m;
    ep.pitch = sp_pitch();
    sp.asp = base; sp.meta = reinterpret_cast<uint8_t *>(meta); sp.ld_a = lay.ld_a; sp.n_rt = lay.n_rt;
    const size_t esmem = sp_expand_smem(geo);
    const int64_t items = lay.n_rt * (SP_ATOM / SP_ROWS_ITEM) * geo.nc;
    const bool aligned = (reinterpret_cast<uintptr_t>(val) & 15) == 0 && (reinterpret_cast<uintptr_t>(idx) & 15) == 0;
    if (dtype == NMG_F16)
        return !aligned ? sp_expand_launch<__half, 0>(sp, esmem, items, st)
               : geo.n == 1 ? sp_expand_launch<__half, 1>(sp, esmem, items, st) : sp_expand_launch<__half, 2>(sp, esmem, items, st);
    return !aligned ? sp_expand_launch<__nv_bfloat16, 0>(sp, esmem, items, st)
           : geo.n == 1 ? sp_expand_launch<__nv_bfloat16, 1>(sp, esmem, items, st) : sp_expand_launch<__nv_bfloat16, 2>(sp, esmem, items, st);
}
size_t tc_sp_copy_bytes(const Geo &geo) { return sp_layout(geo).total; }

// dx[tokens][ld_dx] = dy[tokens][ld_dy] * W from the compressed transposed copy.  dy rows must be 16-byte aligned (TMA).
int tc_sp_matmul_t(const Geo &geo, int dtype, const void *sp_copy, const void *dy, int64_t ld_dy, int64_t tokens, void *dx, int64_t ld_dx,
                   cudaStream_t st) {
    if (!tc_sp_supported(geo, dtype)) NMG_FAIL(NMG_ERR_UNSUPPORTED, "the structured-sparse path needs a 16-bit weight with n <= 2 and m in {4, 8, 16, 32, 64}");
    if (!sp_copy || (reinterpret_cast<uintptr_t>(sp_copy) & 255)) NMG_FAIL(NMG_ERR_INVALID, "the compressed transposed copy must be non-NULL and 256-byte aligned");
    if ((reinterpret_cast<uintptr_t>(dy) & 15) || (ld_dy % 8)) NMG_FAIL(NMG_ERR_UNSUPPORTED, "the structured-sparse path needs 16-byte aligned gradient rows");
    const SpLayout lay = sp_layout(geo);
    const char *base = static_cast<const char *>(sp_copy);
    const char *meta = base + lay.asp_bytes;
    int rc;
    SpGemmMaps maps;
    if ((rc = encode_tmap_2d(&maps.a, dtype, base, (uint64_t)lay.ld_a, (uint64_t)geo.K, (uint64_t)lay.ld_a, 64, TC_BM, 1))) return rc;
    if ((rc = encode_tmap_2d(&maps.b, dtype, dy, (uint64_t)geo.M, (uint64_t)tokens, (uint64_t)ld_dy, TC_BK, 128, 1))) return rc;
    if ((rc = encode_tmap_2d(&maps.e, NMG_F32, meta, 256, (uint64_t)(lay.n_ft * lay.n_rt * 2), 256, 256, 2, 0))) return rc;
    int *status = nullptr;
    if ((rc = get_status_word(&status))) return rc;
    SpGemmParams gp{};
    gp.out = dx;
    gp.out_vec = ((ld_dx * 2) % 16 == 0 && (reinterpret_cast<uintptr_t>(dx) & 15) == 0) ? 1 : 0;
    if (gp.out_vec) {
        if ((rc = encode_tmap_2d(&maps.out, dtype, dx, (uint64_t)geo.K, (uint64_t)tokens, (uint64_t)ld_dx, 32, 32, 0))) return rc;
    } else {
        maps.out = maps.b;  // never used; keeps the parameter defined
    }
    gp.out_feats = geo.K; gp.red = geo.M; gp.ntok = tokens; gp.ld_out = ld_dx; gp.n_rt = lay.n_rt;
    gp.tiles_f = (int)(lay.n_ft / 2);
    gp.tiles_t = (int)((tokens + TC_BN - 1) / TC_BN);
    gp.band = TC_BAND_PAIR;
    {
        // many waves over a long reduction: keep the producers in step; the counter is zeroed in stream order
        int dev = 0, sms = 148;
        NMG_CUDA(cudaGetDevice(&dev));
        NMG_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        if ((int64_t)gp.tiles_f * gp.tiles_t >= 3 * (int64_t)(sms / 2) && geo.M >= 4096) {
            if ((rc = get_wave_counter(&gp.wave_ctr))) return rc;
            NMG_CUDA(cudaMemsetAsync(gp.wave_ctr, 0, sizeof(unsigned), st));
        }
    }
    gp.status = status;
    return dtype == NMG_F16 ? sp_gemm_launch<__half>(gp, maps, st) : sp_gemm_launch<__nv_bfloat16>(gp, maps, st);
}

}  // namespace nmg
