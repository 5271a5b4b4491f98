/*
 * nmg_b200 -- C ABI of the B200 (sm_100a) grouped n:m ("nmg") sparse kernels.
 *
 * This is the boundary a host runtime binds to (ctypes / cffi / cgo / JNI): C linkage, plain pointers
 * and sizes, caller-owned memory, no C++ or framework types.  Every function returns an nmg_status
 * (0 = success); nmg_last_error() gives the message of the calling thread's last failure.  Nothing
 * aborts, nothing throws, and no function synchronises the device: work is queued on the stream the
 * caller passes (a cudaStream_t given as void*, NULL = legacy default stream).
 *
 * Format (2-D view; leading dims of an N-D weight form the batch):
 *   W[M][K] row-major.  n:m blocks run along M (m consecutive rows), groups along K.
 *   C = comb(m,n), cc = C*g, nb = ceil(M/m), nc = ceil(K/cc), tile t = (b*nc + kc)*nb + mb
 *   val[t][p][j][s]  (p < C patterns in revolving-door order, j < g, s < n)   same dtype as W
 *   idx[t][p][j]     int16, position of the column inside its chunk
 * which is exactly the layout of GroupedNMTensor.val / .idx in the reference
 * (src/sten/grouped_nm/grouped_nm_tensor.py:636-655, 877-881).
 *
 * Each entry point names the reference interface it replaces.  The reference compiles one shared
 * object per shape at run time and binds it through ctypes with all-void* signatures; here shapes are
 * arguments of one ahead-of-time library.
 */
#ifndef NMG_B200_H
#define NMG_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum { NMG_F32 = 0, NMG_F16 = 1, NMG_BF16 = 2 } nmg_dtype;

typedef enum {
    NMG_OK = 0,
    NMG_ERR_INVALID = 1,     /* bad argument (shape, pointer, alignment, dtype) */
    NMG_ERR_UNSUPPORTED = 2, /* valid request the library has no kernel for (e.g. tile too large) */
    NMG_ERR_CUDA = 3,        /* a CUDA runtime / driver call failed */
    NMG_ERR_WORKSPACE = 4,   /* workspace missing or too small */
    NMG_ERR_TIMEOUT = 5      /* a bounded device-side wait ran out (see nmg_read_status) */
} nmg_status;

/* Layout of the dense operand of the matmul. */
typedef enum {
    NMG_ACT_TOKEN_MAJOR = 0, /* X[tokens][K] -> Y[tokens][M]   (F.linear: y = x W^T + b) */
    NMG_ACT_K_MAJOR = 1,     /* B[K][tokens] -> C[M][tokens]   (torch.mm:  C = W B)       */
    NMG_ACT_TOKEN_MAJOR_OUT_ROWS = 2 /* X[tokens][K] -> C[M][tokens] (C = W X^T: output rows follow weight rows, so a
                                        row shard of W yields a contiguous row slab of C) */
} nmg_act_layout;

/* Kernel family for nmg_spmm / nmg_spmm_t (NMG_ALGO_AUTO picks by dtype and shape).  NMG_ALGO_TENSOR_DENSE restricts
 * the tensor-core path to the kernels that multiply at the dense rate (no structured-sparse MMA); it only differs from
 * NMG_ALGO_TENSOR for nmg_spmm_t and exists for comparison and measurement. */
typedef enum { NMG_ALGO_AUTO = 0, NMG_ALGO_SIMT = 1, NMG_ALGO_TENSOR = 2, NMG_ALGO_TENSOR_DENSE = 3 } nmg_algo;

int nmg_version(void);
const char *nmg_last_error(void);

/* Number of patterns C = comb(m, n) and the pattern table order[C][n] (int8 row offsets) in the order the
 * format uses.  Replaces make_n_m (grouped_nm_tensor.py:37-50).  Host-only, no CUDA call. */
int64_t nmg_num_patterns(int n, int m);
int nmg_pattern_order(int n, int m, int8_t *order_out);

/* dense -> nmg magnitude sparsifier.  Replaces the generated `func(dense, sparse, idx)` of
 * get_dense_to_grouped_nm_impl_cpu (grouped_nm_tensor.py:220-305; the deterministic CPU result is the parity
 * target) and the four-kernel CUDA version (grouped_nm_tensor.py:356-633), including the pad / permute /
 * contiguous copy of dense_to_grouped_n_m (:701-710): the kernel reads W in place.
 *   dense: [batch][M][K], row stride ld_dense elements, batch stride batch_stride elements.
 *   val, idx: outputs, contiguous, batch*nc*nb tiles.  Selection is done on fp32 magnitudes. */
int nmg_sparsify(const void *dense, int64_t batch, int64_t M, int64_t K, int64_t ld_dense,
                 int64_t batch_stride, int n, int m, int g, int dtype, void *val, int16_t *idx,
                 void *stream);

/* nmg -> dense.  Replaces the generated `func(sparse, dense, idx)` of get_grouped_n_m_to_dense_impl_cpu / _cuda
 * (grouped_nm_tensor.py:713-845) plus the zero-fill and un-merge / un-pad copies of grouped_n_m_to_dense (:848-874).
 * Writes every element of dense[batch][M][K] (zeros included). */
int nmg_densify(const void *val, const int16_t *idx, int64_t batch, int64_t M, int64_t K, int n, int m,
                int g, int dtype, void *dense, int64_t ld_dense, int64_t batch_stride, void *stream);

/* Values of a dense tensor at the positions an EXISTING layout keeps: val[t][p][j][s] = dense[row of slot s of pattern p in
 * tile t][column idx[t][p][j]] (zero outside the tensor).  Replaces GroupedNMTensor.clone_layout
 * (src/sten/grouped_nm/grouped_nm_tensor.py:904-951, disabled there): it is how a gradient or an updated weight takes the
 * layout of the weight it belongs to without a new magnitude selection.  Operand conventions as nmg_sparsify; idx is read,
 * val (same shape and dtype as the layout's val) is written. */
int nmg_gather(const void *dense, const int16_t *idx, int64_t batch, int64_t M, int64_t K, int64_t ld_dense,
               int64_t batch_stride, int n, int m, int g, int dtype, void *val, void *stream);

/* Per-block top-n by magnitude without the group constraint.  Replaces PerfectNMTensor.from_dense / to_dense
 * (src/sten/grouped_nm/grouped_nm_tensor.py:1010-1066: pad, reshape, abs().argsort(descending), gather / scatter_), the
 * upper bound the reference's conversion test compares the grouped layout against (tests/test_nmg.py:73-83).
 * The tensor is [outer][size][inner], contiguous; blocks of m run along `size` (zero-padded to a multiple of m).
 *   val, idx: [outer][ceil(size / m)][n][inner]; idx is int64 (what argsort returns), positions inside the block, ordered
 *   by descending magnitude; equal magnitudes keep the smaller position first (argsort leaves that order open).
 * nmg_perfect_nm_densify writes every element of dense (zeros included). */
int nmg_perfect_nm_select(const void *dense, int64_t outer, int64_t size, int64_t inner, int n, int m, int dtype, void *val,
                          int64_t *idx, void *stream);
int nmg_perfect_nm_densify(const void *val, const int64_t *idx, int64_t outer, int64_t size, int64_t inner, int n, int m,
                           int dtype, void *dense, void *stream);

/* Column-ordered device copy of a weight ("packed" form), the second half of the format conversion: for every
 * row-block and column it holds the column's pattern id and its n kept values, i.e. val / idx re-ordered from
 * pattern-sorted to natural column order.  The tensor-core matmul and the transposed matmul read it; building it
 * once per weight and passing it to nmg_spmm / nmg_spmm_t saves the re-ordering pass of every call.  The copy is
 * an internal cache: it is derived from (val, idx), never serialised, and its layout may change between
 * versions.  No counterpart in the reference (its kernels read val / idx directly).
 *   packed: device buffer of at least nmg_packed_bytes(...) bytes, 256-byte aligned. */
size_t nmg_packed_bytes(int64_t M, int64_t K, int n, int m, int g, int dtype);
int nmg_pack(const void *val, const int16_t *idx, int64_t M, int64_t K, int n, int m, int g, int dtype, void *packed,
             size_t packed_bytes, void *stream);

/* Sparse weight x dense activation.  Replaces `__program_nmg_<hash>(state, A_idx, A_val, B, C, groups)`
 * (src/sten/grouped_nm/sten_impls.py:111-138, generated by dace_gnm_mult.py:572-1007) and the crop / bias add of
 * sparse_torch_nn_functional_linear (sten_impls.py:170-173).
 *   layout NMG_ACT_TOKEN_MAJOR: act = X[tokens][ld_act >= K], out = Y[tokens][ld_out >= M], out = X W^T (+ bias[M])
 *   layout NMG_ACT_K_MAJOR:     act = B[K][ld_act >= tokens], out = C[M][ld_out >= tokens], out = W B (+ bias[M] per row)
 *   layout NMG_ACT_TOKEN_MAJOR_OUT_ROWS: act as TOKEN_MAJOR, out as K_MAJOR
 * act, out, val and bias share `dtype`; accumulation is fp32.  bias may be NULL.
 * packed: result of nmg_pack for the same weight, or NULL (then it is built in the workspace when the chosen kernel
 * needs it).  have_packed in the workspace query says which of the two the caller will do.
 * workspace: device scratch of at least nmg_spmm_workspace_bytes(...) bytes, 256-byte aligned, owned by the
 * caller for the duration of the call (may be NULL when the query returns 0).
 * algo: NMG_ALGO_AUTO uses the tensor cores for token-major activations (16-bit rows must be 16-byte aligned) and
 * weights of at least 64 rows, at every token count; the SIMT kernels otherwise.  Two tensor-core variants exist.  Below 1280 tokens (256 for
 * fp32), for m in {4, 8, 16} and n <= 2, one fused kernel expands tiles of the packed copy inside the matmul.  From
 * there on, and for every other (n, m), the weight is first expanded into a transient dense 16-bit matrix in the workspace
 * (M * round_up(K, 8) * 2 bytes; three such planes for fp32) and multiplied by a persistent TMA-fed kernel; that
 * variant reads val / idx and ignores `packed`.  fp32 operands go through the tensor cores as exact three-way bf16
 * splits with promoted fp32 accumulation (relative error ~3.5e-6, independent of K); NMG_ALGO_SIMT forces plain fp32
 * FMA arithmetic. */
size_t nmg_spmm_workspace_bytes(int64_t M, int64_t K, int64_t tokens, int n, int m, int g, int dtype,
                                int layout, int algo, int have_packed);
int nmg_spmm(const void *val, const int16_t *idx, const void *packed, int64_t M, int64_t K, int n, int m, int g,
             int dtype, const void *act, int64_t ld_act, int64_t tokens, const void *bias, void *out,
             int64_t ld_out, int layout, int algo, void *workspace, size_t workspace_bytes, void *stream);

/* nmg_spmm followed by an activation and a residual add, in one call: out = activation(product + bias) + residual.
 * The reference adds the bias in a separate pass over the output (src/sten/grouped_nm/sten_impls.py:172-173) and leaves
 * activation and residual to the model code; here the two-pass tensor-core matmul applies all three in its epilogue
 * (the output is written once), every other kernel is followed by one elementwise pass.
 *   activation: NMG_EPI_NONE or NMG_EPI_GELU (exact: x/2 * (1 + erf(x / sqrt 2)))
 *   residual:   NULL, or a tensor of the output's shape and orientation with row pitch ld_res.
 * Everything else as nmg_spmm (same workspace query). */
typedef enum { NMG_EPI_NONE = 0, NMG_EPI_GELU = 1 } nmg_epilogue_act;
int nmg_spmm_fused(const void *val, const int16_t *idx, const void *packed, int64_t M, int64_t K, int n, int m, int g,
                   int dtype, const void *act, int64_t ld_act, int64_t tokens, const void *bias, int activation,
                   const void *residual, int64_t ld_res, void *out, int64_t ld_out, int layout, int algo, void *workspace,
                   size_t workspace_bytes, void *stream);

/* Transposed product for the backward pass: dX[tokens][ld_dx >= K] = dY[tokens][ld_dy >= M] * W.
 * The reference has no counterpart (its dispatcher installs a failing backward stub: src/sten/sten.py:1690-1693);
 * the registration shape follows the CSR linear backward (sten.py:2362-2383).
 * Here the weight's rows -- the axis the n:m blocks run along -- are the reduction axis, so for 16-bit weights with
 * n <= 2 and m in {4, 8, 16, 32, 64} (every aligned group of four rows then holds at most two kept values) the tensor
 * cores multiply only the kept values: from 1280 tokens on, NMG_ALGO_AUTO / NMG_ALGO_TENSOR compress W^T into the
 * workspace (two values + two 2-bit positions per group of four rows) and run tcgen05.mma.sp, structured-sparse MMA at
 * twice the dense rate.  fp32 weights, other patterns and fewer tokens use the dense-rate kernels described above. */
size_t nmg_spmm_t_workspace_bytes(int64_t M, int64_t K, int64_t tokens, int n, int m, int g, int dtype,
                                  int algo, int have_packed);
int nmg_spmm_t(const void *val, const int16_t *idx, const void *packed, int64_t M, int64_t K, int n, int m, int g,
               int dtype, const void *dy, int64_t ld_dy, int64_t tokens, void *dx, int64_t ld_dx, int algo,
               void *workspace, size_t workspace_bytes, void *stream);

/* The transposed product from a compressed transposed copy the caller keeps ("sp24": W^T with two stored values and two
 * 2-bit positions per aligned group of four weight rows, in the tensor core's 2:4 operand layout).  nmg_spmm_t builds
 * this copy in its workspace on every call; a caller that runs many backward passes on one weight builds it once with
 * nmg_pack_sp24 and calls nmg_spmm_t_sp24, which launches the structured-sparse matmul alone.  The copy is an internal
 * cache like the packed copy: derived from (val, idx), never serialised, layout may change between versions.
 * nmg_sp24_bytes returns 0 when the weight is outside the structure (fp32, n > 2, m not in {4, 8, 16, 32, 64}).
 * sp24 must be 256-byte aligned; dy rows 16-byte aligned.  No counterpart in the reference (it has no backward). */
size_t nmg_sp24_bytes(int64_t M, int64_t K, int n, int m, int g, int dtype);
int nmg_pack_sp24(const void *val, const int16_t *idx, int64_t M, int64_t K, int n, int m, int g, int dtype, void *sp24,
                  size_t sp24_bytes, void *stream);
int nmg_spmm_t_sp24(const void *sp24, int64_t M, int64_t K, int n, int m, int g, int dtype, const void *dy, int64_t ld_dy,
                    int64_t tokens, void *dx, int64_t ld_dx, void *stream);

/* Opt-in for compute-bound serving: keep the EXPANDED 16-bit weight across calls.  From 1280 tokens on nmg_spmm expands
 * the weight into its workspace on every call (about M * K * 2.5 bytes of HBM traffic); a caller that prefers speed over
 * the format's memory saving expands once (nmg_expand: M * round_up(K, 8) * 2 bytes) and calls nmg_spmm_expanded, which
 * runs the tensor-core matmul and the fused epilogue of nmg_spmm_fused alone.  The counterpart of the kernel-choice knob
 * of GroupedNMTensor.set_spmm_opt (src/sten/grouped_nm/grouped_nm_tensor.py:892-902); off unless asked for.
 * 16-bit dtypes, token-major activations with 16-byte aligned rows; `expanded` 256-byte aligned. */
size_t nmg_expanded_bytes(int64_t M, int64_t K, int n, int m, int g, int dtype);
int nmg_expand(const void *val, const int16_t *idx, int64_t M, int64_t K, int n, int m, int g, int dtype, void *expanded,
               size_t expanded_bytes, void *stream);
int nmg_spmm_expanded(const void *expanded, int64_t M, int64_t K, int dtype, const void *act, int64_t ld_act, int64_t tokens,
                      const void *bias, int activation, const void *residual, int64_t ld_res, void *out, int64_t ld_out,
                      int layout, void *stream);

/* Whether nmg_spmm (transposed = 0) or nmg_spmm_t (transposed = 1) would read the packed copy for this problem under
 * `algo`, assuming aligned operands: 1 or 0.  Lets a host build and keep packed copies only for the weights and batch
 * sizes that use them (the two-pass tensor-core variant and the SIMT forward kernel do not).  `layout` is ignored for
 * transposed = 1.  No counterpart in the reference. */
int nmg_spmm_uses_packed(int64_t M, int64_t K, int64_t tokens, int n, int m, int g, int dtype, int layout, int algo,
                         int transposed);

/* Row-shard matmul fused with the exchange of its result: C = W X^T (+ bias per row), C[M][ld_out >= tokens], written
 * by the matmul kernel's epilogue into EVERY buffer of outs[0 .. n_outs) with 128-byte coalesced stores.  outs[0] is
 * the caller's own buffer; the others are the same location of the same buffer on peer GPUs, mapped into this
 * process (CUDA IPC or a symmetric-memory allocation), so that a row-sharded layer needs no all-gather: when every
 * rank's call has completed, every GPU holds the full C.  The caller synchronises the ranks afterwards (any
 * stream-ordered collective or barrier).  Operand conventions as nmg_spmm with NMG_ACT_TOKEN_MAJOR_OUT_ROWS; workspace
 * of nmg_spmm_replicated_workspace_bytes(...) bytes.  Always runs on the two-pass tensor-core variant:
 * NMG_ERR_UNSUPPORTED for unaligned 16-bit activation rows or a chunk that does not fit shared memory.  At most 8 buffers.  No counterpart in the reference, which has no multi-GPU path for this format. */
size_t nmg_spmm_replicated_workspace_bytes(int64_t M, int64_t K, int64_t tokens, int n, int m, int g, int dtype);
int nmg_spmm_replicated(const void *val, const int16_t *idx, int64_t M, int64_t K, int n, int m, int g, int dtype,
                        const void *act, int64_t ld_act, int64_t tokens, const void *bias, void *const *outs, int n_outs,
                        void *multicast_out, int64_t ld_out, void *workspace, size_t workspace_bytes, void *stream);

/* Matmul for callers that cannot allocate device memory (no counterpart in the reference, whose host code allocates
 * every buffer with torch: src/sten/grouped_nm/grouped_nm_tensor.py:652-672, sten_impls.py:127).
 * Meant for code that runs where cudaMalloc is not an option: under CUDA-graph capture or another stream-ordered
 * region, in a server that partitioned all of HBM up front, in a callback that may not take allocator locks.
 * Same arguments and result as nmg_spmm with NMG_ALGO_SIMT, minus the workspace: the scratch (fp32 re-layout of the
 * activation, 256 + K * round_up(tokens, 128) * 4 bytes) lives in a fixed device array inside the library.
 *   - limit: that size must not exceed NMG_NOALLOC_SCRATCH_BYTES, else NMG_ERR_UNSUPPORTED (nothing is truncated);
 *     only n:m in {1:4, 2:4, 1:8, 2:8, 1:16, 3:6} are served (others need an allocated pattern table);
 *   - every GPU that loads the library holds the array until the process exits;
 *   - all calls on a device share it: calls that overlap in time on one GPU race and must be serialised by the caller;
 *   - the first call on a device resolves the array's address and clears its status word (synchronous); make
 *     it before any stream capture begins;
 *   - its kernels report a bounded wait that ran out in the first word of that array, not in the allocated status
 *     word of the other entry points; nmg_read_status reads both and itself allocates nothing.
 * Calls no cudaMalloc / cudaFree and no allocating library routine. */
#define NMG_NOALLOC_SCRATCH_BYTES (32u << 20)
int nmg_spmm_noalloc(const void *val, const int16_t *idx, int64_t M, int64_t K, int n, int m, int g, int dtype,
                     const void *act, int64_t ld_act, int64_t tokens, const void *bias, void *out, int64_t ld_out,
                     int layout, void *stream);

/* Measurement helpers (no counterpart in the reference; its profiling is wall-clock around whole operators,
 * src/sten/sten.py:30-49).
 * nmg_profile_next: the next nmg_spmm / nmg_spmm_t call made by this thread records `start_event` immediately before
 * and `stop_event` immediately after its dominant kernel (the one that does the multiply-adds), on the call's
 * stream.  Both are cudaEvent_t handles passed as void*; the request is consumed by that one call.
 * nmg_measure_fma_peak: runs an unrolled, dependency-free FFMA loop on every SM and returns the sustained fp32
 * multiply-add rate in TFLOP/s: the roofline of the SIMT kernels.  Synchronises the stream. */
int nmg_profile_next(void *start_event, void *stop_event);
int nmg_measure_fma_peak(double *tflops_out, void *stream);

/* Pitched asynchronous copy between host and device (or device and device): `rows` rows of `width_bytes` bytes,
 * row pitches dst_pitch / src_pitch bytes, queued on `stream`.  A host helper for pipelines that move a column block
 * of a row-major matrix (a token chunk of C[M][tokens]) between pinned host memory and the GPU while other chunks
 * compute; the direction is inferred from the pointers.  No counterpart in the reference. */
int nmg_memcpy_2d_async(void *dst, size_t dst_pitch, const void *src, size_t src_pitch, size_t width_bytes, size_t rows,
                        void *stream);

/* Device-side status of the kernels launched so far on the current device: 0 when every bounded wait completed, else
 * the code of a wait that ran out (returned as NMG_ERR_TIMEOUT, and cleared).  Covers the status word of the
 * workspace-taking entry points and the one nmg_spmm_noalloc keeps in its built-in array.  Synchronises the given
 * stream; allocates nothing. */
int nmg_read_status(void *stream, int *status_out);

/* Self-test of the bounded device-side waits (no counterpart in the reference, whose kernels have no waits): launches a
 * one-CTA kernel whose only thread waits on an mbarrier that nothing arrives at, with the same bounded wait every kernel
 * of the library uses but a limit of `limit_ns` nanoseconds (1 .. 1e9).  The wait runs out, the kernel records code 90 in
 * the status word and returns normally; the next nmg_read_status reports NMG_ERR_TIMEOUT once and clears it.  Nothing
 * faults or hangs: this is how the time-out path is exercised. */
int nmg_selftest_wait(uint64_t limit_ns, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* NMG_B200_H */
