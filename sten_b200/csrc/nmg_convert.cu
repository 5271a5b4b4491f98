// Format conversion kernels: dense -> nmg magnitude sparsifier (bit-exact with the sequential definition of the
// format) and nmg -> dense.  Both are one pass over the weight; the weight is read / written in place in its
// [batch][M][K] layout, so no padded, permuted or zero-filled temporaries exist.
#include "nmg_common.cuh"

namespace nmg {

// =====================================================================================================
// Sparsifier.
//
// Definition of the result (the reference's CPU implementation): for every tile, score each (column c, pattern p)
// with the fp32 sum of |w| over the rows of p (summed in slot order), sort all (score, c, p) triples
// descending (ties: larger c, then larger p) and walk the list once, accepting a triple when its column is
// still free and its pattern holds fewer than g columns.
//
// That walk is a greedy matching of columns (capacity 1) to patterns (capacity g) by descending weight under a strict
// total order of the pairs.  Such a matching is the unique stable one: the heaviest pair must be matched in any stable
// matching (otherwise it blocks), remove it and repeat.  Deferred acceptance reaches the same matching in a few parallel
// rounds instead of C*g sequential steps: every free column proposes to the best pattern it can still enter, every
// pattern keeps its g best proposers (sorted by (score, c) descending) and releases the rest, released columns propose
// again.  A pattern's final list in descending order is exactly the order in which the sequential walk accepted its
// columns, so val / idx come out bit for bit identical -- without the C^2*g-element sort, without a sequential chain of
// C*g dependent reductions, and without scratch memory in HBM.
//
// One warp per tile.  Lanes own columns (c = lane, lane + 32, ...) when columns propose, and patterns (p = lane,
// lane + 32, ...) when patterns merge their proposers.  The tile is read with 16-byte loads where alignment allows.
// =====================================================================================================

// (row-block, column chunk, batch entry) of a tile; 32-bit division whenever the tile count allows it (a 64-bit division
// costs about as much as scoring a column).
__device__ __forceinline__ void tile_coords(int64_t tile, int64_t nb, int64_t nc, int64_t tiles, int64_t &mb, int64_t &kc, int64_t &b) {
    if (tiles < 0x7fffffffll) {
        const unsigned t = (unsigned)tile, unb = (unsigned)nb, unc = (unsigned)nc;
        const unsigned q = t / unb;
        mb = t - q * unb;
        const unsigned q2 = q / unc;
        kc = q - q2 * unc;
        b = q2;
    } else {
        mb = tile % nb;
        kc = (tile / nb) % nc;
        b = tile / (nb * nc);
    }
}

struct SparsifyParams {
    const void *dense;
    void *val;
    int16_t *idx;
    const int8_t *order;  // [C][n] device
    int64_t M, K, ld, batch_stride;
    int64_t nb, nc, tiles;
    int n, m, g, C, cc;
    int slab_bytes;  // shared memory per warp
};

// A proposal / list entry: fp32 score bits (non-negative, so unsigned order = float order) above the column index.
// Comparing entries of one pattern as integers is the format's order (score, then larger column first).
__device__ __forceinline__ uint64_t sp_key(uint32_t score_bits, int c) { return ((uint64_t)score_bits << 16) | (uint32_t)c; }

// Shared memory of one warp (host and device agree through this function).
struct SparsifySlab { size_t list, inbox, x, park, state, prop_p, prop_i, cnt, total; };
__host__ __device__ inline SparsifySlab sparsify_slab(int m, int cc, int C, size_t es) {
    SparsifySlab l;
    size_t o = 0;
    l.list = o;   o += (size_t)cc * 8;                                   // [C][g] kept proposers of every pattern, descending
    l.inbox = o;  o += (size_t)cc * 8;                                   // [cc] this round's proposals, grouped by pattern
    l.x = o;      o += (((size_t)m * cc * es) + 15) & ~(size_t)15;       // [m][cc] the tile
    l.park = o;   o += (size_t)cc * 4;                                   // [cc] score of the column's proposal
    l.state = o;  o += (size_t)cc * 2;                                   // [cc] pattern the column is held by, -1 = free
    l.prop_p = o; o += (size_t)cc * 2;                                   // [cc] pattern proposed to this round
    l.prop_i = o; o += (size_t)cc * 2;                                   // [cc] position inside that pattern's inbox segment
    o = (o + 3) & ~(size_t)3;
    l.cnt = o;    o += (size_t)C * 4 * 3;                                // [C] list lengths, proposals this round, segment starts
    l.total = (o + 15) & ~(size_t)15;
    return l;
}


// Zero phase of the selection.  Triples whose score is 0 come last in the format's order, sorted by larger column, then
// larger pattern; when the walk reaches them every pattern in which a still-free column scores above zero is full.  So
// the free columns, taken from the largest index down, each fill the largest pattern that has room left: a closed form,
// no rounds.  (Zero-padded columns of a last chunk and all-zero columns of a pruned weight end up here; letting them
// run through the rounds would cost one round per pattern with hundreds of tied proposals each.)
// On entry cnt[p] holds the list lengths; rem / cum are scratch of C ints each.  All lanes of the warp call this.
__device__ __forceinline__ void sparsify_zero_phase(int lane, int cc, int C, int g, uint64_t *list, int16_t *state, int *cnt, int *rem, int *cum) {
    // cum[p] = free places in patterns with a larger index (suffix sum), rem[p] = free places of p
    const int pchunk = (C + 31) / 32;
    const int p0 = lane * pchunk, p1 = min(C, p0 + pchunk);
    int local = 0;
    for (int p = p0; p < p1; p++) { rem[p] = g - cnt[p]; local += g - cnt[p]; }
    int incl = local;  // inclusive suffix sum over lanes
    for (int d = 1; d < 32; d <<= 1) {
        const int t = __shfl_down_sync(0xffffffffu, incl, d);
        if (lane + d < 32) incl += t;
    }
    int run = incl - local;  // free places in the chunks of higher lanes
    for (int p = p1 - 1; p >= p0; p--) { cum[p] = run; run += g - cnt[p]; }
    __syncwarp();
    int above = 0;  // free columns in higher rows of the column-to-lane layout (larger indices), warp-uniform
    for (int k = (cc - 1) / 32; k >= 0; k--) {
        const int c = k * 32 + lane;
        const bool is_free = c < cc && state[c] < 0;
        const uint32_t mask = __ballot_sync(0xffffffffu, is_free);
        if (is_free) {
            const int i = above + __popc(lane == 31 ? 0u : (mask >> (lane + 1)));  // free columns with a larger index
            int lo = 0, hi = C - 1;  // largest p with cum[p] <= i (cum decreases with p, cum[C - 1] = 0)
            while (lo < hi) {
                const int mid = (lo + hi) >> 1;
                if (cum[mid] <= i) hi = mid; else lo = mid + 1;
            }
            // patterns without room share their cum with the next smaller pattern that has some: step down to it
            int p = lo;
            while (p > 0 && i - cum[p] >= rem[p]) p--;
            list[p * g + cnt[p] + (i - cum[p])] = (uint64_t)(uint32_t)c;  // score 0
            state[c] = (int16_t)p;
        }
        above += __popc(mask);
    }
    __syncwarp();
}

template <typename T>
__global__ void __launch_bounds__(256) sparsify_kernel(SparsifyParams prm) {
    extern __shared__ __align__(16) char smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int n = prm.n, m = prm.m, g = prm.g, C = prm.C, cc = prm.cc;
    constexpr int V = 16 / (int)sizeof(T);  // elements per 16-byte access

    // CTA-wide copy of the pattern table, then one slab per warp.
    int8_t *ord = reinterpret_cast<int8_t *>(smem);
    const int ord_bytes = (C * n + 15) & ~15;
    for (int i = threadIdx.x; i < C * n; i += blockDim.x) ord[i] = prm.order[i];
    __syncthreads();

    char *slab = smem + ord_bytes + (size_t)warp * prm.slab_bytes;
    const SparsifySlab lay = sparsify_slab(m, cc, C, sizeof(T));
    uint64_t *list = reinterpret_cast<uint64_t *>(slab + lay.list);
    uint64_t *inbox = reinterpret_cast<uint64_t *>(slab + lay.inbox);
    T *x = reinterpret_cast<T *>(slab + lay.x);
    uint32_t *park = reinterpret_cast<uint32_t *>(slab + lay.park);
    int16_t *state = reinterpret_cast<int16_t *>(slab + lay.state);
    int16_t *prop_p = reinterpret_cast<int16_t *>(slab + lay.prop_p);
    int16_t *prop_i = reinterpret_cast<int16_t *>(slab + lay.prop_i);
    int *cnt = reinterpret_cast<int *>(slab + lay.cnt);
    int *icnt = cnt + C;
    int *ioff = icnt + C;

    const T *dense = static_cast<const T *>(prm.dense);
    T *val = static_cast<T *>(prm.val);
    const int pchunk = (C + 31) / 32;  // patterns per lane in the prefix sum

    for (int64_t tile = (int64_t)blockIdx.x * nwarps + warp; tile < prm.tiles; tile += (int64_t)gridDim.x * nwarps) {
        int64_t mb, kc, b;
        tile_coords(tile, prm.nb, prm.nc, prm.tiles, mb, kc, b);
        const int64_t row0 = mb * m, col0 = kc * cc;
        const T *src = dense + b * prm.batch_stride;
        // ---- load the tile (rows beyond M and columns beyond K read as zero)
        const bool full_cols = col0 + cc <= prm.K;
        for (int r = 0; r < m; r++) {
            const bool row_ok = row0 + r < prm.M;
            const T *srow = src + (row0 + r) * prm.ld + col0;
            T *xr = x + r * cc;
            if (row_ok && full_cols && (cc % V) == 0 && (reinterpret_cast<uintptr_t>(srow) & 15) == 0) {
                for (int c = lane * V; c < cc; c += 32 * V)
                    *reinterpret_cast<uint4 *>(xr + c) = __ldg(reinterpret_cast<const uint4 *>(srow + c));
            } else {
                for (int c = lane; c < cc; c += 32) xr[c] = (row_ok && col0 + c < prm.K) ? srow[c] : DT<T>::from_f32(0.f);
            }
        }
        for (int c = lane; c < cc; c += 32) state[c] = -1;
        for (int p = lane; p < C; p += 32) cnt[p] = 0;
        __syncwarp();

        // ---- deferred acceptance.  Every round with a free column makes at least one proposal (column, pattern) that was
        // never made before, so cc * C rounds cannot be exceeded; real weights settle in a handful.
        for (int round = 0; round < cc * C + 2; round++) {
            for (int p = lane; p < C; p += 32) icnt[p] = 0;
            __syncwarp();
            // columns propose: the best pattern (larger p on equal score) among those the column can still enter
            bool proposed = false;
            for (int c = lane; c < cc; c += 32) {
                prop_p[c] = -1;
                if (state[c] >= 0) continue;
                uint32_t best_s = 0;
                int best_p = -1;
                for (int p = 0; p < C; p++) {
                    float s = 0.f;
                    for (int i = 0; i < n; i++) s = __fadd_rn(s, fabsf(DT<T>::to_f32(x[(int)ord[p * n + i] * cc + c])));
                    const uint32_t sb = __float_as_uint(s);
                    if (sb == 0) continue;  // zero scores are placed by the closed form after the rounds
                    if (cnt[p] >= g && sp_key(sb, c) <= list[p * g + g - 1]) continue;  // full, and every kept proposer ranks higher
                    if (best_p < 0 || sb >= best_s) { best_s = sb; best_p = p; }
                }
                if (best_p < 0) continue;  // nothing above zero is open to this column: it waits for the zero phase
                proposed = true;
                prop_p[c] = (int16_t)best_p;
                prop_i[c] = (int16_t)atomicAdd(&icnt[best_p], 1);
                park[c] = best_s;
            }
            if (!__any_sync(0xffffffffu, proposed)) break;
            __syncwarp();
            // exclusive prefix sum of the proposal counts -> start of every pattern's inbox segment
            {
                const int p0 = lane * pchunk, p1 = min(C, p0 + pchunk);
                int local = 0;
                for (int p = p0; p < p1; p++) local += icnt[p];
                int incl = local;
                for (int d = 1; d < 32; d <<= 1) {
                    const int t = __shfl_up_sync(0xffffffffu, incl, d);
                    if (lane >= d) incl += t;
                }
                int run = incl - local;
                for (int p = p0; p < p1; p++) { ioff[p] = run; run += icnt[p]; }
            }
            __syncwarp();
            for (int c = lane; c < cc; c += 32)
                if (prop_p[c] >= 0) inbox[ioff[prop_p[c]] + prop_i[c]] = sp_key(park[c], c);
            __syncwarp();
            // patterns merge their proposers into their sorted lists; what does not fit is released
            for (int p = lane; p < C; p += 32) {
                uint64_t *lp = list + p * g;
                int L = cnt[p];
                const int e0 = ioff[p], e1 = e0 + icnt[p];
                for (int e = e0; e < e1; e++) {
                    const uint64_t key = inbox[e];
                    if (L == g) {
                        if (key <= lp[g - 1]) continue;            // stays free (state is still -1)
                        state[(int)(lp[g - 1] & 0xffffu)] = -1;     // the weakest kept proposer is released
                        L = g - 1;
                    }
                    int j = L;
                    while (j > 0 && lp[j - 1] < key) { lp[j] = lp[j - 1]; j--; }
                    lp[j] = key;
                    L++;
                    state[(int)(key & 0xffffu)] = (int16_t)p;
                }
                cnt[p] = L;
            }
            __syncwarp();
        }
        __syncwarp();
        sparsify_zero_phase(lane, cc, C, g, list, state, cnt, icnt, ioff);

        // ---- write the tile: idx = the lists' columns, val = the kept rows of those columns
        int16_t *idx_out = prm.idx + tile * cc;
        T *val_out = val + tile * (int64_t)cc * n;
        for (int s0 = lane; s0 < cc; s0 += 32) idx_out[s0] = (int16_t)(list[s0] & 0xffffu);
        for (int e = lane; e < cc * n; e += 32) {
            const int s0 = e / n, t = e - s0 * n;
            const int c = (int)(list[s0] & 0xffffu), p = s0 / g;
            val_out[e] = x[(int)ord[p * n + t] * cc + c];
        }
        __syncwarp();
    }
}

// Shared memory of one warp in the (n, m)-specialised kernel: no copy of the tile (its values are re-read through L1),
// lists as separate score / column arrays, proposals as column indices.  8.3 KB for a 448-column tile, so that about
// twenty-seven warps are resident per SM: the selection is a chain of dependent shared-memory accesses, and residency is what hides it.
struct SparsifyLean { size_t lscore, park, lcol, inbox, state, prop_p, freel, cnt, total; };
__host__ __device__ inline SparsifyLean sparsify_lean(int cc, int C) {
    SparsifyLean l;
    size_t o = 0;
    l.lscore = o; o += (size_t)cc * 4;   // [C][g] score bits of the kept proposers, descending by (score, column)
    l.park = o;   o += (size_t)cc * 4;   // [cc] score of the column's current proposal / match
    l.lcol = o;   o += (size_t)cc * 2;   // [C][g] their columns
    l.inbox = o;  o += (size_t)cc * 2;   // [cc] this round's proposing columns, grouped by pattern
    l.state = o;  o += (size_t)cc * 2;   // [cc] pattern the column is held by, -1 = free
    l.prop_p = o; o += (size_t)cc * 2;   // [cc] pattern proposed to this round, -1 = none
    l.freel = o;  o += (size_t)cc * 2;   // columns that propose in the next round (rejected or released in this one)
    o = (o + 3) & ~(size_t)3;
    l.cnt = o;    o += (size_t)C * 4 * 3 + 4;  // cnt, icnt, ioff per pattern + the length of freel
    l.total = (o + 15) & ~(size_t)15;
    return l;
}

// Specialisation on (n, m): the pattern table is a compile-time constant, so a column's |w| values sit in registers and
// all C scores are straight-line adds; which patterns are full is one bit mask (C <= 32), so the first round -- where
// nothing is full -- touches no shared state at all.  The first round's proposals are placed by rank (every proposal
// counts the larger proposals of its own pattern, all lanes busy) instead of by one lane per pattern inserting in turn.
template <int N_, int M_, typename T>
__global__ void __launch_bounds__(256, 4) sparsify_nm_kernel(SparsifyParams prm) {
    extern __shared__ __align__(16) char smem[];
    constexpr Order<N_, M_> ORD{};
    constexpr int C = Order<N_, M_>::C;
    static_assert(C <= 32, "the full-pattern mask is one word");
    constexpr int V = 16 / (int)sizeof(T);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int g = prm.g, cc = prm.cc;

    int8_t *ord = reinterpret_cast<int8_t *>(smem);  // run-time copy of the table for the output stage
    constexpr int ord_bytes = (C * N_ + 15) & ~15;
    for (int i = threadIdx.x; i < C * N_; i += blockDim.x) ord[i] = (int8_t)ORD.v[(i / N_) * Order<N_, M_>::LD + (i % N_)];
    __syncthreads();

    char *slab = smem + ord_bytes + (size_t)warp * prm.slab_bytes;
    const SparsifyLean lay = sparsify_lean(cc, C);
    uint32_t *lscore = reinterpret_cast<uint32_t *>(slab + lay.lscore);
    uint32_t *park = reinterpret_cast<uint32_t *>(slab + lay.park);
    int16_t *lcol = reinterpret_cast<int16_t *>(slab + lay.lcol);
    int16_t *inbox = reinterpret_cast<int16_t *>(slab + lay.inbox);
    int16_t *state = reinterpret_cast<int16_t *>(slab + lay.state);
    int16_t *prop_p = reinterpret_cast<int16_t *>(slab + lay.prop_p);
    int16_t *freel = reinterpret_cast<int16_t *>(slab + lay.freel);
    int *cnt = reinterpret_cast<int *>(slab + lay.cnt);
    int *icnt = cnt + C;
    int *ioff = icnt + C;
    int *nfree = ioff + C;

    const T *dense = static_cast<const T *>(prm.dense);
    T *val = static_cast<T *>(prm.val);
    const bool g_pow2 = (g & (g - 1)) == 0;
    const int g_shift = 31 - __clz(g);
    // (score, column) order of the format: larger score first, on equal scores the larger column
    auto above = [](uint32_t s1, int c1, uint32_t s2, int c2) { return s1 > s2 || (s1 == s2 && c1 > c2); };

    for (int64_t tile = (int64_t)blockIdx.x * nwarps + warp; tile < prm.tiles; tile += (int64_t)gridDim.x * nwarps) {
        int64_t mb, kc, b;
        tile_coords(tile, prm.nb, prm.nc, prm.tiles, mb, kc, b);
        const int64_t row0 = mb * M_, col0 = kc * cc;
        const T *src = dense + b * prm.batch_stride + row0 * prm.ld + col0;  // element (r, c) of the tile at src[r * ld + c]
        const int rows_ok = (int)(prm.M - row0 < M_ ? prm.M - row0 : M_);    // rows beyond M and columns beyond K read as zero
        const int cols_ok = (int)(prm.K - col0 < cc ? prm.K - col0 : cc);
        auto tile_at = [&](int r, int c) -> T { return (r < rows_ok && c < cols_ok) ? __ldg(src + (int64_t)r * prm.ld + c) : DT<T>::from_f32(0.f); };

        for (int c = lane; c < cc; c += 32) state[c] = -1;
        if (lane < C) cnt[lane] = 0;
        uint32_t full_mask = 0;  // bit p: pattern p holds g columns (warp-uniform)
        __syncwarp();

        // Deferred acceptance.  Every round with a proposal makes at least one (column, pattern) proposal that was never
        // made before, so cc * C rounds cannot be exceeded; real weights settle in a handful.
        // After the first round only the columns that were rejected or released propose again: they are kept as a list, so
        // that a late round with a handful of free columns costs a handful of iterations, not a sweep over the tile.
        for (int round = 0; round < cc * C + 2; round++) {
            const int F = round == 0 ? cc : *nfree;  // proposers of this round: every column, then the list
            if (lane < C) icnt[lane] = 0;
            __syncwarp();
            if (lane == 0) *nfree = 0;
            bool proposed = false;
            for (int e = lane; e < F; e += 32) {
                const int c = round == 0 ? e : (int)freel[e];
                prop_p[c] = -1;
                float a[M_];
#pragma unroll
                for (int r = 0; r < M_; r++) a[r] = fabsf(DT<T>::to_f32(tile_at(r, c)));
                uint32_t best_s = 0;  // a score of zero never wins: zero scores are placed by the closed form after the rounds
                int best_p = -1;
                if (full_mask == 0) {  // first round(s): every pattern is open, nothing but registers
                    // the sum starts from the first value (0 + x = x exactly for x >= 0) and zero scores are sorted out once,
                    // after the scan: a zero maximum means that every score of the column is zero
#pragma unroll
                    for (int p = 0; p < C; p++) {
                        float sc = a[ORD.row(p, 0)];
#pragma unroll
                        for (int i = 1; i < N_; i++) sc = __fadd_rn(sc, a[ORD.row(p, i)]);
                        const uint32_t sb = __float_as_uint(sc);
                        if (sb >= best_s) { best_s = sb; best_p = p; }
                    }
                    if (best_s == 0) best_p = -1;
                } else {
#pragma unroll
                    for (int p = 0; p < C; p++) {
                        float sc = a[ORD.row(p, 0)];
#pragma unroll
                        for (int i = 1; i < N_; i++) sc = __fadd_rn(sc, a[ORD.row(p, i)]);
                        const uint32_t sb = __float_as_uint(sc);
                        bool open = sb != 0 && sb >= best_s;
                        // full pattern: only a proposer that ranks above its weakest kept one gets in
                        if (open && ((full_mask >> p) & 1u)) open = above(sb, c, lscore[p * g + g - 1], lcol[p * g + g - 1]);
                        if (open) { best_s = sb; best_p = p; }
                    }
                }
                if (best_p < 0) continue;  // nothing above zero is open to this column: it waits for the zero phase
                proposed = true;
                prop_p[c] = (int16_t)best_p;
                park[c] = best_s;
                atomicAdd(&icnt[best_p], 1);
            }
            if (!__any_sync(0xffffffffu, proposed)) break;
            __syncwarp();
            int total;
            {   // exclusive prefix sum over the patterns (one per lane) -> start of every pattern's inbox segment
                const int mine = lane < C ? icnt[lane] : 0;
                int incl = mine;
#pragma unroll
                for (int d = 1; d < 32; d <<= 1) {
                    const int t = __shfl_up_sync(0xffffffffu, incl, d);
                    if (lane >= d) incl += t;
                }
                if (lane < C) { ioff[lane] = incl - mine; icnt[lane] = 0; }  // icnt becomes the fill cursor of the segment
                total = __shfl_sync(0xffffffffu, incl, 31);
            }
            __syncwarp();
            for (int e = lane; e < F; e += 32) {
                const int c = round == 0 ? e : (int)freel[e];
                const int p = prop_p[c];
                if (p >= 0) inbox[ioff[p] + atomicAdd(&icnt[p], 1)] = (int16_t)c;
            }
            __syncwarp();  // the list has been read: the steps below refill it
            if (round == 0) {
                // all lists are empty: a proposal's place is its rank among the proposals of its pattern
                for (int e = lane; e < total; e += 32) {
                    const int c = inbox[e], p = prop_p[c];
                    const uint32_t sc = park[c];
                    const int e0 = ioff[p], e1 = e0 + icnt[p];
                    int rank = 0;
                    for (int j = e0; j < e1; j++) {
                        const int c2 = inbox[j];
                        rank += above(park[c2], c2, sc, c) ? 1 : 0;
                    }
                    if (rank < g) { lscore[p * g + rank] = sc; lcol[p * g + rank] = (int16_t)c; state[c] = (int16_t)p; }
                    else freel[atomicAdd(nfree, 1)] = (int16_t)c;
                }
                if (lane < C) cnt[lane] = min(icnt[lane], g);
            } else if (lane < C) {
                const int p = lane;
                uint32_t *ls = lscore + p * g;
                int16_t *lc = lcol + p * g;
                int L = cnt[p];
                const int e0 = ioff[p], e1 = e0 + icnt[p];
                for (int e = e0; e < e1; e++) {
                    const int c = inbox[e];
                    const uint32_t sc = park[c];
                    if (L == g) {
                        if (!above(sc, c, ls[g - 1], lc[g - 1])) {  // stays free
                            freel[atomicAdd(nfree, 1)] = (int16_t)c;
                            continue;
                        }
                        state[lc[g - 1]] = -1;                          // the weakest kept proposer is released
                        freel[atomicAdd(nfree, 1)] = lc[g - 1];
                        L = g - 1;
                    }
                    int j = L;
                    while (j > 0 && above(sc, c, ls[j - 1], lc[j - 1])) { ls[j] = ls[j - 1]; lc[j] = lc[j - 1]; j--; }
                    ls[j] = sc;
                    lc[j] = (int16_t)c;
                    L++;
                    state[c] = (int16_t)p;
                }
                cnt[p] = L;
            }
            __syncwarp();
            full_mask = __ballot_sync(0xffffffffu, lane < C && cnt[lane] == g);
        }
        __syncwarp();
        // zero phase on the split lists: same closed form as sparsify_zero_phase, columns only
        {
            const int mine = lane < C ? g - cnt[lane] : 0;  // free places of pattern `lane`
            int incl = mine;                                 // inclusive suffix sum over lanes
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int t = __shfl_down_sync(0xffffffffu, incl, d);
                if (lane + d < 32) incl += t;
            }
            if (lane < C) { icnt[lane] = mine; ioff[lane] = incl - mine; }  // rem[p], cum[p] = free places in larger patterns
            __syncwarp();
            int above_cnt = 0;
            for (int k = (cc - 1) / 32; k >= 0; k--) {
                const int c = k * 32 + lane;
                const bool is_free = c < cc && state[c] < 0;
                const uint32_t mask = __ballot_sync(0xffffffffu, is_free);
                if (is_free) {
                    const int i = above_cnt + __popc(lane == 31 ? 0u : (mask >> (lane + 1)));  // free columns with a larger index
                    int p = C - 1;
                    while (p > 0 && ioff[p] + icnt[p] <= i) p--;  // largest pattern whose range of places contains i
                    lcol[p * g + cnt[p] + (i - ioff[p])] = (int16_t)c;
                    state[c] = (int16_t)p;
                }
                above_cnt += __popc(mask);
            }
            __syncwarp();
        }

        int16_t *idx_out = prm.idx + tile * cc;
        T *val_out = val + tile * (int64_t)cc * N_;
        if ((cc & 7) == 0 && (reinterpret_cast<uintptr_t>(idx_out) & 15) == 0) {
            for (int s0 = lane * 8; s0 < cc; s0 += 256) *reinterpret_cast<uint4 *>(idx_out + s0) = *reinterpret_cast<const uint4 *>(lcol + s0);
        } else {
            for (int s0 = lane; s0 < cc; s0 += 32) idx_out[s0] = lcol[s0];
        }
        const int nvals = cc * N_;
        if ((nvals % V) == 0 && (reinterpret_cast<uintptr_t>(val_out) & 15) == 0) {
            for (int v = lane * V; v < nvals; v += 32 * V) {
                __align__(16) T out[V];
#pragma unroll
                for (int u = 0; u < V; u++) {
                    const int e = v + u, s0 = e / N_, t = e % N_;
                    const int c = lcol[s0], p = g_pow2 ? (s0 >> g_shift) : s0 / g;
                    out[u] = tile_at((int)ord[p * N_ + t], c);
                }
                *reinterpret_cast<uint4 *>(val_out + v) = *reinterpret_cast<const uint4 *>(out);
            }
        } else {
            for (int e = lane; e < nvals; e += 32) {
                const int s0 = e / N_, t = e % N_;
                const int c = lcol[s0], p = s0 / g;
                val_out[e] = tile_at((int)ord[p * N_ + t], c);
            }
        }
        __syncwarp();
    }
}

// =====================================================================================================
// Densifier: one CTA per tile.  The tile's idx is inverted in shared memory (column -> slot), val is staged,
// and the m x cc block is written row by row with coalesced stores; zeros are produced by the same stores, so
// the output needs no separate clearing pass.
// =====================================================================================================
struct DensifyParams {
    const void *val;
    const int16_t *idx;
    void *dense;
    const int8_t *slot_of_row;  // [C][m] device
    int64_t M, K, ld, batch_stride;
    int64_t nb, nc, tiles;
    int n, m, g, C, cc;
};

template <typename T>
__global__ void __launch_bounds__(128) densify_kernel(DensifyParams prm) {
    extern __shared__ __align__(16) char smem[];
    const int n = prm.n, m = prm.m, g = prm.g, C = prm.C, cc = prm.cc;
    T *sval = reinterpret_cast<T *>(smem);                                             // [cc][n]
    int16_t *pos = reinterpret_cast<int16_t *>(smem + (((size_t)cc * n * sizeof(T) + 15) & ~(size_t)15));  // [cc]
    int8_t *sor = reinterpret_cast<int8_t *>(pos + cc);                                // [C][m]
    for (int i = threadIdx.x; i < C * m; i += blockDim.x) sor[i] = prm.slot_of_row[i];

    const T *val = static_cast<const T *>(prm.val);
    T *dense = static_cast<T *>(prm.dense);
    for (int64_t tile = blockIdx.x; tile < prm.tiles; tile += gridDim.x) {
        int64_t mb, kc, b;
        tile_coords(tile, prm.nb, prm.nc, prm.tiles, mb, kc, b);
        __syncthreads();
        for (int c = threadIdx.x; c < cc; c += blockDim.x) pos[c] = -1;
        constexpr int V = 16 / (int)sizeof(T);  // elements per 16-byte access
        const T *vsrc = val + tile * (int64_t)cc * n;
        if (((cc * n) % V) == 0 && (reinterpret_cast<uintptr_t>(vsrc) & 15) == 0) {
            for (int e = threadIdx.x * V; e < cc * n; e += blockDim.x * V)
                *reinterpret_cast<uint4 *>(sval + e) = __ldg(reinterpret_cast<const uint4 *>(vsrc + e));
        } else {
            for (int e = threadIdx.x; e < cc * n; e += blockDim.x) sval[e] = vsrc[e];
        }
        __syncthreads();
        const int16_t *isrc = prm.idx + tile * cc;
        if ((cc & 7) == 0 && (reinterpret_cast<uintptr_t>(isrc) & 15) == 0) {
            for (int s8 = threadIdx.x * 8; s8 < cc; s8 += blockDim.x * 8) {
                const uint4 iv = __ldg(reinterpret_cast<const uint4 *>(isrc + s8));
                const int16_t *ci = reinterpret_cast<const int16_t *>(&iv);
#pragma unroll
                for (int u = 0; u < 8; u++)
                    if (ci[u] >= 0 && ci[u] < cc) pos[ci[u]] = (int16_t)(s8 + u);  // a malformed index is ignored, never dereferenced
            }
        } else {
            for (int s = threadIdx.x; s < cc; s += blockDim.x) {
                const int c = isrc[s];
                if (c >= 0 && c < cc) pos[c] = (int16_t)s;
            }
        }
        __syncthreads();
        T *dst = dense + b * prm.batch_stride;
        const int64_t col0 = kc * cc;
        // 16-byte stores where the row piece allows it: every thread assembles V consecutive columns of one row
        const bool vec = (cc % V) == 0 && col0 + cc <= prm.K && (prm.ld % V) == 0 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0;
        if (vec) {
            const int per_row = cc / V;
            for (int v = threadIdx.x; v < m * per_row; v += blockDim.x) {
                const int r = v / per_row, c0 = (v - r * per_row) * V;
                const int64_t row = mb * m + r;
                if (row >= prm.M) continue;
                __align__(16) T out[V];
#pragma unroll
                for (int u = 0; u < V; u++) {
                    const int sl = pos[c0 + u];
                    T val_u = DT<T>::from_f32(0.f);
                    if (sl >= 0) {
                        const int t = sor[(sl / g) * m + r];
                        if (t >= 0) val_u = sval[sl * n + t];
                    }
                    out[u] = val_u;
                }
                *reinterpret_cast<uint4 *>(dst + row * prm.ld + col0 + c0) = *reinterpret_cast<const uint4 *>(out);
            }
            continue;
        }
        for (int r = 0; r < m; r++) {
            const int64_t row = mb * m + r;
            if (row >= prm.M) break;
            T *drow = dst + row * prm.ld + kc * cc;
            for (int c = threadIdx.x; c < cc; c += blockDim.x) {
                if (kc * cc + c >= prm.K) break;
                const int s = pos[c];
                T v = DT<T>::from_f32(0.f);
                if (s >= 0) {
                    const int t = sor[(s / g) * m + r];
                    if (t >= 0) v = sval[s * n + t];
                }
                drow[c] = v;
            }
        }
    }
}

// =====================================================================================================
// Layout gather: the values of a dense tensor at the positions an existing (idx) layout keeps.  One warp per tile; the
// tile's rows are short contiguous spans, so the indexed reads hit L1 / L2.
// =====================================================================================================
struct GatherParams {
    const void *dense;
    const int16_t *idx;
    void *val;
    const int8_t *order;  // [C][n] device
    int64_t M, K, ld, batch_stride;
    int64_t nb, nc, tiles;
    int n, m, g, C, cc;
};

template <typename T>
__global__ void __launch_bounds__(256) gather_layout_kernel(GatherParams prm) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int n = prm.n, m = prm.m, g = prm.g, cc = prm.cc;
    const T *dense = static_cast<const T *>(prm.dense);
    T *val = static_cast<T *>(prm.val);
    for (int64_t tile = (int64_t)blockIdx.x * nwarps + warp; tile < prm.tiles; tile += (int64_t)gridDim.x * nwarps) {
        int64_t mb, kc, b;
        tile_coords(tile, prm.nb, prm.nc, prm.tiles, mb, kc, b);
        const T *src = dense + b * prm.batch_stride;
        const int16_t *isrc = prm.idx + tile * cc;
        T *vdst = val + tile * (int64_t)cc * n;
        for (int s = lane; s < cc; s += 32) {
            const int c = isrc[s];
            const int8_t *o = prm.order + (s / g) * n;
            const int64_t col = kc * cc + c;
            const bool col_ok = c >= 0 && c < cc && col < prm.K;  // a malformed index reads as zero, never dereferenced
            for (int t = 0; t < n; t++) {
                const int64_t row = mb * m + o[t];
                vdst[s * n + t] = (col_ok && row < prm.M) ? src[row * prm.ld + col] : DT<T>::from_f32(0.f);
            }
        }
    }
}

static int sm_count() {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    return sms > 0 ? sms : 148;
}

static int check_dtype(int dtype) {
    if (dtype != NMG_F32 && dtype != NMG_F16 && dtype != NMG_BF16)
        NMG_FAIL(NMG_ERR_INVALID, "dtype must be NMG_F32, NMG_F16 or NMG_BF16, got %d", dtype);
    return NMG_OK;
}

}  // namespace nmg

using namespace nmg;

extern "C" int nmg_sparsify(const void *dense, int64_t batch, int64_t M, int64_t K, int64_t ld_dense,
                            int64_t batch_stride, int n, int m, int g, int dtype, void *val, int16_t *idx,
                            void *stream) {
    Geo geo;
    int rc = make_geo(M, K, n, m, g, &geo);
    if (rc) return rc;
    if ((rc = check_dtype(dtype))) return rc;
    if (!dense || !val || !idx) NMG_FAIL(NMG_ERR_INVALID, "dense, val and idx must be non-NULL");
    if (n < 1) NMG_FAIL(NMG_ERR_INVALID, "the sparsifier needs n >= 1");
    if (batch < 1 || ld_dense < K || (batch > 1 && batch_stride < M * ld_dense))
        NMG_FAIL(NMG_ERR_INVALID, "bad batch / leading dimension (batch=%lld ld=%lld)", (long long)batch, (long long)ld_dense);
    PatternTable tab;
    if ((rc = get_pattern_table(n, m, &tab))) return rc;

    SparsifyParams p{};
    p.dense = dense; p.val = val; p.idx = idx; p.order = tab.order;
    p.M = M; p.K = K; p.ld = ld_dense; p.batch_stride = batch_stride;
    p.nb = geo.nb; p.nc = geo.nc; p.tiles = batch * geo.nb * geo.nc;
    p.n = n; p.m = m; p.g = g; p.C = geo.C; p.cc = geo.cc;
    const bool specialised = (n == 1 && (m == 4 || m == 8 || m == 16)) || (n == 2 && (m == 4 || m == 8));
    const size_t slab = specialised ? sparsify_lean(geo.cc, geo.C).total : sparsify_slab(m, geo.cc, geo.C, dtype_size(dtype)).total;
    const size_t ord_bytes = ((size_t)geo.C * n + 15) & ~(size_t)15;
    const size_t budget = 200 * 1024;
    if (ord_bytes + slab > budget)
        NMG_FAIL(NMG_ERR_UNSUPPORTED, "tile of m=%d x %d columns needs %zu bytes of shared memory (limit %zu)", m, geo.cc,
                 ord_bytes + slab, budget);
    // warps per CTA: whatever keeps the most warps resident per SM (227 KB of shared memory, at most 8 warps per CTA); on a
    // tie the smaller CTA, for a finer tail
    int warps = 1, best_resident = 0;
    for (int w = 1; w <= 8; w++) {
        const size_t per_cta = ord_bytes + (size_t)w * slab + 1024;  // + the per-CTA reservation of the driver
        if (per_cta > 227 * 1024) break;
        int per_sm = (int)((size_t)227 * 1024 / per_cta);
        if (per_sm > 32) per_sm = 32;
        if (per_sm * w > 64) per_sm = 64 / w;
        if (per_sm * w > best_resident) { best_resident = per_sm * w; warps = w; }
    }
    p.slab_bytes = (int)slab;
    const size_t smem = ord_bytes + warps * slab;
    int64_t ctas = (p.tiles + warps - 1) / warps;
    const int64_t max_ctas = (int64_t)sm_count() * 16;
    if (ctas > max_ctas) ctas = max_ctas;
    cudaStream_t st = (cudaStream_t)stream;
    bool launched = false;
#define NMG_SPARSIFY_CASE(N_, M_)                                                                                     \
    if (!launched && n == N_ && m == M_) {                                                                            \
        NMG_DISPATCH_DTYPE(dtype, T, {                                                                                \
            NMG_CUDA(cudaFuncSetAttribute(sparsify_nm_kernel<N_, M_, T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
            sparsify_nm_kernel<N_, M_, T><<<(unsigned)ctas, warps * 32, smem, st>>>(p);                               \
        });                                                                                                           \
        launched = true;                                                                                              \
    }
    NMG_SPARSIFY_CASE(1, 4)
    NMG_SPARSIFY_CASE(2, 4)
    NMG_SPARSIFY_CASE(1, 8)
    NMG_SPARSIFY_CASE(2, 8)
    NMG_SPARSIFY_CASE(1, 16)
#undef NMG_SPARSIFY_CASE
    if (!launched) {
        NMG_DISPATCH_DTYPE(dtype, T, {
            NMG_CUDA(cudaFuncSetAttribute(sparsify_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            sparsify_kernel<T><<<(unsigned)ctas, warps * 32, smem, st>>>(p);
        });
    }
    NMG_CUDA(cudaGetLastError());
    return NMG_OK;
}

extern "C" int nmg_densify(const void *val, const int16_t *idx, int64_t batch, int64_t M, int64_t K, int n, int m,
                           int g, int dtype, void *dense, int64_t ld_dense, int64_t batch_stride, void *stream) {
    Geo geo;
    int rc = make_geo(M, K, n, m, g, &geo);
    if (rc) return rc;
    if ((rc = check_dtype(dtype))) return rc;
    if (!dense || !val || !idx) NMG_FAIL(NMG_ERR_INVALID, "dense, val and idx must be non-NULL");
    if (batch < 1 || ld_dense < K || (batch > 1 && batch_stride < M * ld_dense))
        NMG_FAIL(NMG_ERR_INVALID, "bad batch / leading dimension (batch=%lld ld=%lld)", (long long)batch, (long long)ld_dense);
    cudaStream_t st = (cudaStream_t)stream;
    // Aligned outputs go through the weight-expansion pass of the matmul path (tiles scattered in shared memory, 16-byte
    // stores that also write the zeros); the kernel below serves the rest.
    if (tc_expand_plain_supported(geo, dtype, dense, ld_dense) && (batch == 1 || batch_stride % 8 == 0)) {
        const size_t es0 = dtype_size(dtype);
        const int64_t tiles1 = geo.nb * geo.nc;
        for (int64_t b = 0; b < batch; b++) {
            const char *vb = static_cast<const char *>(val) + (size_t)b * tiles1 * geo.cc * n * es0;
            if ((rc = tc_expand_plain(geo, dtype, vb, idx + b * tiles1 * geo.cc, static_cast<char *>(dense) + (size_t)b * batch_stride * es0, ld_dense, st)))
                return rc;
        }
        return NMG_OK;
    }
    PatternTable tab;
    if ((rc = get_pattern_table(n, m, &tab))) return rc;

    DensifyParams p{};
    p.val = val; p.idx = idx; p.dense = dense; p.slot_of_row = tab.slot_of_row;
    p.M = M; p.K = K; p.ld = ld_dense; p.batch_stride = batch_stride;
    p.nb = geo.nb; p.nc = geo.nc; p.tiles = batch * geo.nb * geo.nc;
    p.n = n; p.m = m; p.g = g; p.C = geo.C; p.cc = geo.cc;
    const size_t es = dtype_size(dtype);
    const size_t smem = (((size_t)geo.cc * n * es + 15) & ~(size_t)15) + (size_t)geo.cc * 2 + (size_t)geo.C * m;
    if (smem > 200 * 1024)
        NMG_FAIL(NMG_ERR_UNSUPPORTED, "tile of %d columns needs %zu bytes of shared memory (limit %d)", geo.cc, smem, 200 * 1024);
    int64_t ctas = p.tiles;
    const int64_t max_ctas = (int64_t)sm_count() * 32;
    if (ctas > max_ctas) ctas = max_ctas;
    NMG_DISPATCH_DTYPE(dtype, T, {
        NMG_CUDA(cudaFuncSetAttribute(densify_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        densify_kernel<T><<<(unsigned)ctas, 128, smem, st>>>(p);
    });
    NMG_CUDA(cudaGetLastError());
    return NMG_OK;
}

extern "C" int nmg_gather(const void *dense, const int16_t *idx, int64_t batch, int64_t M, int64_t K, int64_t ld_dense,
                          int64_t batch_stride, int n, int m, int g, int dtype, void *val, void *stream) {
    Geo geo;
    int rc = make_geo(M, K, n, m, g, &geo);
    if (rc) return rc;
    if ((rc = check_dtype(dtype))) return rc;
    if (!dense || !val || !idx) NMG_FAIL(NMG_ERR_INVALID, "dense, val and idx must be non-NULL");
    if (n < 1) NMG_FAIL(NMG_ERR_INVALID, "n must be >= 1");
    if (batch < 1 || ld_dense < K || (batch > 1 && batch_stride < M * ld_dense))
        NMG_FAIL(NMG_ERR_INVALID, "bad batch / leading dimension (batch=%lld ld=%lld)", (long long)batch, (long long)ld_dense);
    PatternTable tab;
    if ((rc = get_pattern_table(n, m, &tab))) return rc;
    GatherParams p{};
    p.dense = dense; p.idx = idx; p.val = val; p.order = tab.order;
    p.M = M; p.K = K; p.ld = ld_dense; p.batch_stride = batch_stride;
    p.nb = geo.nb; p.nc = geo.nc; p.tiles = batch * geo.nb * geo.nc;
    p.n = n; p.m = m; p.g = g; p.C = geo.C; p.cc = geo.cc;
    int64_t ctas = (p.tiles + 7) / 8;
    const int64_t max_ctas = (int64_t)sm_count() * 16;
    if (ctas > max_ctas) ctas = max_ctas;
    cudaStream_t st = (cudaStream_t)stream;
    NMG_DISPATCH_DTYPE(dtype, T, { gather_layout_kernel<T><<<(unsigned)ctas, 256, 0, st>>>(p); });
    NMG_CUDA(cudaGetLastError());
    return NMG_OK;
}
