// Specialised SIMT transposed kernel (template) and its launcher; instantiated per (n, m) in nmg_bwd_inst_*.cu.
#pragma once
#include "nmg_spmm_simt.cuh"

namespace nmg {

// ------------------------------------------------------------------------------------------ specialised kernel
template <int N_, int M_, int P>
__device__ __forceinline__ void bwd_apply(float (&acc)[kBwdTT], const float (&dy)[M_][kBwdTT], const float (&w)[N_]) {
    constexpr Order<N_, M_> ORD{};
#pragma unroll
    for (int s = 0; s < N_; s++)
#pragma unroll
        for (int t = 0; t < kBwdTT; t++) acc[t] = fmaf(w[s], dy[ORD.row(P, s)][t], acc[t]);
}

#define NMG_BWD_CASE(P) \
    case P:             \
        if constexpr (P < C) bwd_apply<N_, M_, P>(acc[kk], dy, w); \
        break;

template <int N_, int M_, typename T>
__global__ void __launch_bounds__(kBwdWarps * 32, 1)
spmm_bwd_simt_kernel(const BwdParams prm, const __grid_constant__ CUtensorMap tmap) {
    constexpr int C = Order<N_, M_>::C;
    static_assert(C <= 32, "switch below covers 32 patterns");
    static_assert((kColsCta * N_ * sizeof(T)) % 16 == 0, "value slab rows must be 16-byte multiples");
    extern __shared__ char smem_raw[];
    char *smem = reinterpret_cast<char *>(((uintptr_t)smem_raw + 127) & ~(uintptr_t)127);
    const int RS = prm.rb_stage;
    const BwdSmemPlan plan = bwd_smem_plan(M_, N_, RS, sizeof(T));
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + 2 * plan.stage_bytes);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t tok0 = (int64_t)blockIdx.x * kBwdTok;
    const int64_t k0 = (int64_t)blockIdx.y * kColsCta;
    const int64_t nsteps = (prm.nb + RS - 1) / RS;
    const T *nval = static_cast<const T *>(prm.nval);

    if (tid == 0) {
        mbar_init(&full[0], 1);
        mbar_init(&full[1], 1);
        mbar_fence_init();
    }
    __syncthreads();

    auto issue = [&](int64_t step, int st) {
        char *base = smem + plan.stage_bytes * st;
        const int64_t mb_first = step * RS;
        const int nrb = (int)((prm.nb - mb_first) < RS ? (prm.nb - mb_first) : RS);
        if (tid == 0) {
            mbar_expect_tx(&full[st], (uint32_t)plan.y_bytes);
            // one box of RS*M_ rows of dY^T (rows past M are zero-filled by TMA)
            tma_load_2d(base, &tmap, (int)tok0, (int)(mb_first * M_), &full[st]);
        }
        // pattern / value slabs: per row-block one 128-column run, 16-byte aligned because the copy is 128 wide
        char *ps = base + plan.y_bytes;
        char *vs = base + plan.y_bytes + plan.p_bytes;
        constexpr int PB = kColsCta * 2 / 16, VB = kColsCta * N_ * (int)sizeof(T) / 16;  // 16-byte blocks per row-block
        for (int e = tid; e < nrb * PB; e += kBwdWarps * 32) {
            const int rb = e / PB, b = e - rb * PB;
            cp_async_16(ps + (size_t)e * 16, reinterpret_cast<const char *>(prm.pat + (mb_first + rb) * prm.Kp + k0) + b * 16);
        }
        for (int e = tid; e < nrb * VB; e += kBwdWarps * 32) {
            const int rb = e / VB, b = e - rb * VB;
            cp_async_16(vs + (size_t)e * 16, reinterpret_cast<const char *>(nval + ((mb_first + rb) * prm.Kp + k0) * N_) + b * 16);
        }
        cp_async_commit();
    };

    float acc[kKW][kBwdTT];
#pragma unroll
    for (int kk = 0; kk < kKW; kk++)
#pragma unroll
        for (int t = 0; t < kBwdTT; t++) acc[kk][t] = 0.f;

    issue(0, 0);
    for (int64_t step = 0; step < nsteps; step++) {
        const int st = (int)(step & 1);
        __syncthreads();  // stage st^1 was fully consumed in the previous iteration; slabs of stage st are written
        if (step + 1 < nsteps) {
            issue(step + 1, st ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        const bool ok = mbar_wait_bounded(&full[st], (uint32_t)((step >> 1) & 1), prm.status, 2);
        if (!__syncthreads_and(ok)) return;

        const char *base = smem + plan.stage_bytes * st;
        const float *Ys = reinterpret_cast<const float *>(base);
        const uint16_t *ps = reinterpret_cast<const uint16_t *>(base + plan.y_bytes);
        const T *vs = reinterpret_cast<const T *>(base + plan.y_bytes + plan.p_bytes);
        const int64_t mb_first = step * RS;
        const int nrb = (int)((prm.nb - mb_first) < RS ? (prm.nb - mb_first) : RS);
        for (int rb = 0; rb < nrb; rb++) {
            float dy[M_][kBwdTT];
#pragma unroll
            for (int r = 0; r < M_; r++) {
                const float4 v = *reinterpret_cast<const float4 *>(Ys + (size_t)(rb * M_ + r) * kBwdTok + lane * kBwdTT);
                dy[r][0] = v.x; dy[r][1] = v.y; dy[r][2] = v.z; dy[r][3] = v.w;
            }
            const uint16_t *pw = ps + rb * kColsCta + warp * kKW;
            const T *vw = vs + (size_t)(rb * kColsCta + warp * kKW) * N_;
#pragma unroll
            for (int kk = 0; kk < kKW; kk++) {
                const int p = pw[kk];
                float w[N_];
#pragma unroll
                for (int s = 0; s < N_; s++) w[s] = DT<T>::to_f32(vw[kk * N_ + s]);
                switch (p) {
                    NMG_BWD_CASE(0) NMG_BWD_CASE(1) NMG_BWD_CASE(2) NMG_BWD_CASE(3) NMG_BWD_CASE(4) NMG_BWD_CASE(5)
                    NMG_BWD_CASE(6) NMG_BWD_CASE(7) NMG_BWD_CASE(8) NMG_BWD_CASE(9) NMG_BWD_CASE(10) NMG_BWD_CASE(11)
                    NMG_BWD_CASE(12) NMG_BWD_CASE(13) NMG_BWD_CASE(14) NMG_BWD_CASE(15) NMG_BWD_CASE(16) NMG_BWD_CASE(17)
                    NMG_BWD_CASE(18) NMG_BWD_CASE(19) NMG_BWD_CASE(20) NMG_BWD_CASE(21) NMG_BWD_CASE(22) NMG_BWD_CASE(23)
                    NMG_BWD_CASE(24) NMG_BWD_CASE(25) NMG_BWD_CASE(26) NMG_BWD_CASE(27) NMG_BWD_CASE(28) NMG_BWD_CASE(29)
                    NMG_BWD_CASE(30) NMG_BWD_CASE(31)
                    default: break;
                }
            }
        }
    }

    T *dx = static_cast<T *>(prm.dx);
#pragma unroll
    for (int t = 0; t < kBwdTT; t++) {
        const int64_t tok = tok0 + lane * kBwdTT + t;
        if (tok >= prm.ntok) continue;
#pragma unroll
        for (int kk = 0; kk < kKW; kk++) {
            const int64_t k = k0 + warp * kKW + kk;
            if (k < prm.K) dx[tok * prm.ld_dx + k] = DT<T>::from_f32(acc[kk][t]);
        }
    }
}

template <int N_, int M_, typename T>
int launch_bwd(const BwdParams &p, const CUtensorMap &tm, int64_t tokens, cudaStream_t st) {
    const size_t smem = bwd_smem_plan(M_, N_, p.rb_stage, sizeof(T)).total;
    dim3 grid((unsigned)((tokens + kBwdTok - 1) / kBwdTok), (unsigned)((p.K + kColsCta - 1) / kColsCta));
    if (grid.y > 65535) NMG_FAIL(NMG_ERR_UNSUPPORTED, "weight has too many columns for one launch");
    NMG_CUDA(cudaFuncSetAttribute(spmm_bwd_simt_kernel<N_, M_, T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    spmm_bwd_simt_kernel<N_, M_, T><<<grid, kBwdWarps * 32, smem, st>>>(p, tm);
    NMG_CUDA(cudaGetLastError());
    return NMG_OK;
}


template <int N_, int M_>
int simt_bwd_launch(int dtype, const BwdParams &p, const CUtensorMap &tm, int64_t tokens, cudaStream_t st) {
    NMG_DISPATCH_DTYPE(dtype, T, return (launch_bwd<N_, M_, T>(p, tm, tokens, st)));
}

}  // namespace nmg
