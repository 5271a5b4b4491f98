// Specialised SIMT forward kernel (template) and its launcher; instantiated per (n, m) in nmg_fwd_inst_*.cu so the
// instances compile in parallel.
#pragma once
#include "nmg_spmm_simt.cuh"

namespace nmg {

// ------------------------------------------------------------------------------------------ specialised forward kernel
template <int TT> struct VecLoad;
template <> struct VecLoad<4> {
    __device__ static __forceinline__ void ld(const float *p, float (&x)[4]) {
        float4 v = *reinterpret_cast<const float4 *>(p);
        x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
    }
};
template <> struct VecLoad<2> {
    __device__ static __forceinline__ void ld(const float *p, float (&x)[2]) {
        float2 v = *reinterpret_cast<const float2 *>(p);
        x[0] = v.x; x[1] = v.y;
    }
};
template <> struct VecLoad<1> {
    __device__ static __forceinline__ void ld(const float *p, float (&x)[1]) { x[0] = *p; }
};
template <> struct VecLoad<8> {
    __device__ static __forceinline__ void ld(const float *p, float (&x)[8]) {
        float4 a = *reinterpret_cast<const float4 *>(p), b = *reinterpret_cast<const float4 *>(p + 4);
        x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
    }
};

template <int M_> struct RowBlocksPerWarp { static constexpr int value = 16 / M_ > 0 ? 16 / M_ : 1; };

template <int N_, int M_, int TT, typename T, bool TOKEN_MAJOR_OUT>
__global__ void __launch_bounds__(kWarps * 32, 1)
spmm_fwd_simt_kernel(const FwdParams prm, const __grid_constant__ CUtensorMap tmap) {
    constexpr Order<N_, M_> ORD{};
    constexpr int C = Order<N_, M_>::C;
    constexpr int RBW = RowBlocksPerWarp<M_>::value;
    constexpr int RBC = kWarps * RBW;
    constexpr int TOKC = 32 * TT;

    extern __shared__ char smem_raw[];
    char *smem = reinterpret_cast<char *>(((uintptr_t)smem_raw + 127) & ~(uintptr_t)127);
    const int cc = prm.cc, g = prm.g;
    const FwdSmemPlan plan = fwd_smem_plan(cc, N_, RBC, TOKC, prm.nbox, prm.box_rows, sizeof(T), prm.stages);
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + plan.stage_bytes * prm.stages);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t tok0 = (int64_t)blockIdx.x * TOKC;
    const int64_t mb0 = (int64_t)blockIdx.y * RBC;
    const int nrb = (int)((prm.nb - mb0) < RBC ? (prm.nb - mb0) : RBC);

    if (tid == 0) {
        mbar_init(&full[0], 1);
        mbar_init(&full[1], 1);
        mbar_fence_init();
    }
    __syncthreads();

    const T *gval = static_cast<const T *>(prm.val);
    auto issue = [&](int64_t kc, int st) {
        char *base = smem + plan.stage_bytes * st;
        if (tid == 0) {
            mbar_expect_tx(&full[st], (uint32_t)plan.x_bytes);
            for (int b = 0; b < prm.nbox; b++)
                tma_load_2d(base + (size_t)b * prm.box_rows * TOKC * 4, &tmap, (int)tok0, (int)(kc * cc + b * prm.box_rows), &full[st]);
        }
        const int64_t t0 = kc * prm.nb + mb0;
        stage_bytes_async(base + plan.x_bytes, gval + t0 * cc * N_, (int64_t)nrb * cc * N_ * sizeof(T), tid, kWarps * 32);
        stage_bytes_async(base + plan.x_bytes + plan.v_bytes, prm.idx + t0 * cc, (int64_t)nrb * cc * 2, tid, kWarps * 32);
        cp_async_commit();
    };

    float acc[RBW][M_][TT];
#pragma unroll
    for (int a = 0; a < RBW; a++)
#pragma unroll
        for (int r = 0; r < M_; r++)
#pragma unroll
            for (int t = 0; t < TT; t++) acc[a][r][t] = 0.f;

    const bool two = prm.stages == 2;
    issue(0, 0);
    for (int64_t kc = 0; kc < prm.nc; kc++) {
        const int st = two ? (int)(kc & 1) : 0;
        const bool more = kc + 1 < prm.nc;
        if (two && more) {
            issue(kc + 1, st ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        const uint32_t parity = two ? (uint32_t)((kc >> 1) & 1) : (uint32_t)(kc & 1);
        const bool ok = mbar_wait_bounded(&full[st], parity, prm.status, 1);
        if (!__syncthreads_and(ok)) return;  // a TMA never landed: status word is set, leave without storing

        const float *Xs = reinterpret_cast<const float *>(smem + plan.stage_bytes * st);
        // the slabs keep their global 16-byte phase in shared memory (see stage_bytes_async)
        const int64_t t0 = kc * prm.nb + mb0;
        const char *sbase = smem + plan.stage_bytes * st + plan.x_bytes;
        const T *vs = reinterpret_cast<const T *>(sbase + ((uintptr_t)(gval + t0 * cc * N_) & 15));
        const int16_t *is = reinterpret_cast<const int16_t *>(sbase + plan.v_bytes + ((uintptr_t)(prm.idx + t0 * cc) & 15));
#pragma unroll
        for (int a = 0; a < RBW; a++) {
            const int mbl = warp * RBW + a;
            if (mbl < nrb) {
                const T *v = vs + (size_t)mbl * cc * N_;
                const int16_t *ix = is + (size_t)mbl * cc;
#pragma unroll
                for (int p = 0; p < C; p++) {
                    const int base = p * g;
#pragma unroll 4
                    for (int j = 0; j < g; j++) {
                        const unsigned k = min((unsigned)(int)ix[base + j], (unsigned)(cc - 1));
                        float x[TT];
                        VecLoad<TT>::ld(Xs + (size_t)k * TOKC + lane * TT, x);
#pragma unroll
                        for (int s = 0; s < N_; s++) {
                            const float w = DT<T>::to_f32(v[(base + j) * N_ + s]);
#pragma unroll
                            for (int t = 0; t < TT; t++) acc[a][ORD.row(p, s)][t] = fmaf(w, x[t], acc[a][ORD.row(p, s)][t]);
                        }
                    }
                }
            }
        }
        __syncthreads();
        if (!two && more) issue(kc + 1, 0);
    }

    // ---- epilogue: bias, convert, store
    T *out = static_cast<T *>(prm.out);
    const T *bias = static_cast<const T *>(prm.bias);
#pragma unroll
    for (int a = 0; a < RBW; a++) {
        const int mbl = warp * RBW + a;
        if (mbl >= nrb) continue;
        const int64_t row0 = (mb0 + mbl) * M_;
#pragma unroll
        for (int r = 0; r < M_; r++) {
            const int64_t row = row0 + r;
            if (row >= prm.M) continue;
            const float b = bias ? DT<T>::to_f32(bias[row]) : 0.f;
#pragma unroll
            for (int t = 0; t < TT; t++) {
                const int64_t tok = tok0 + lane * TT + t;
                if (tok >= prm.ntok) continue;
                const T o = DT<T>::from_f32(acc[a][r][t] + b);
                if (TOKEN_MAJOR_OUT) out[tok * prm.ld_out + row] = o;
                else out[row * prm.ld_out + tok] = o;
            }
        }
    }
}

template <int N_, int M_, int TT, typename T>
int launch_fwd(const FwdParams &p, const CUtensorMap &tm, int rbc, size_t smem, bool token_major, int64_t tokens, cudaStream_t st) {
    dim3 grid((unsigned)((tokens + 32 * TT - 1) / (32 * TT)), (unsigned)((p.nb + rbc - 1) / rbc));
    if (grid.y > 65535) NMG_FAIL(NMG_ERR_UNSUPPORTED, "weight has too many row-blocks for one launch");
    if (token_major) {
        NMG_CUDA(cudaFuncSetAttribute(spmm_fwd_simt_kernel<N_, M_, TT, T, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        spmm_fwd_simt_kernel<N_, M_, TT, T, true><<<grid, kWarps * 32, smem, st>>>(p, tm);
    } else {
        NMG_CUDA(cudaFuncSetAttribute(spmm_fwd_simt_kernel<N_, M_, TT, T, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        spmm_fwd_simt_kernel<N_, M_, TT, T, false><<<grid, kWarps * 32, smem, st>>>(p, tm);
    }
    NMG_CUDA(cudaGetLastError());
    return NMG_OK;
}

template <int N_, int M_, typename T>
int launch_fwd_tt(int tt, const FwdParams &p, const CUtensorMap &tm, int rbc, size_t smem, bool token_major, int64_t tokens, cudaStream_t st) {
    switch (tt) {
        case 4: return launch_fwd<N_, M_, 4, T>(p, tm, rbc, smem, token_major, tokens, st);
        case 2: return launch_fwd<N_, M_, 2, T>(p, tm, rbc, smem, token_major, tokens, st);
        default: return launch_fwd<N_, M_, 1, T>(p, tm, rbc, smem, token_major, tokens, st);
    }
}


template <int N_, int M_>
int simt_fwd_launch(int dtype, int tt, const FwdParams &p, const CUtensorMap &tm, int rbc, size_t smem, bool token_major,
                    int64_t tokens, cudaStream_t st) {
    NMG_DISPATCH_DTYPE(dtype, T, return (launch_fwd_tt<N_, M_, T>(tt, p, tm, rbc, smem, token_major, tokens, st)));
}

}  // namespace nmg
