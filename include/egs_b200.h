/*
 * egs_b200.h - C ABI of the B200 (sm_100a) fused expert gather / scatter library (libegs_b200.so).
 *
 * Every entry point takes raw device pointers, explicit sizes and a CUDA stream, launches on that
 * stream and returns without synchronising.  Return value: 0 on success, otherwise one of the
 * EGS_ERR_* codes below (text: egs_status_string).  No entry point allocates device memory, and the
 * library keeps no device state besides what the caller passes in, unless its comment says so.
 *
 * Tensor layouts (all contiguous, row-major), as in the reference (README.md:7-9):
 *     X / Out / dX : [B, T, I]        rows addressed by token id t in [0, T)
 *     Y / dY       : [B, E, K, J]
 *     Ind          : [B, E, K]        integer token ids, 16/32/64 bit
 *     W            : [E, C, N] or [E, N, C] (see w_layout), C = contracted width, N = produced width
 *
 * The three operators and the six places the reference uses them (egs/triton_kernels.py):
 *     G  gather-GEMM   : gather forward (:367-392)        and scatter backward dY  (:500-508)
 *     S  GEMM-scatter  : scatter forward (:449-474)       and gather backward dX   (:416-424)
 *     D  weight grad   : gather backward dW (:431-439)    and scatter backward dW  (:515-523)
 */
#ifndef EGS_B200_H_
#define EGS_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Element types; the numbering is the reference's dtype_to_type_id (egs/triton_kernels.py:15-23). */
enum { EGS_F32 = 0, EGS_F16 = 1, EGS_BF16 = 2 };
/* Index element types of Ind (the reference's tests pass int16, test_all.py:16; benchmarks int64). */
enum { EGS_I16 = 0, EGS_I32 = 1, EGS_I64 = 2 };
/* Arithmetic for float32 tensors.  STRICT reproduces IEEE-like float32 products (the reference runs
 * its dots with allow_tf32=False, egs/triton_kernels.py:389): on the tensor-core path it is the
 * three-product TF32 split.  TF32 is one TF32 product.  Ignored for 16-bit tensors (fp32 accumulate). */
enum { EGS_PREC_STRICT = 0, EGS_PREC_TF32 = 1 };
/* Kernel family.  AUTO picks the tcgen05 tensor-core kernels when the shape is eligible (row pitches
 * multiples of 16 bytes, 16-byte aligned bases) and the generic CUDA-core kernels otherwise. */
enum { EGS_PATH_AUTO = 0, EGS_PATH_GENERIC = 1, EGS_PATH_TENSOR = 2,
       /* egs_gather_gemm / egs_gather_gemm_bias only, 16-bit tensors, N a multiple of 32 and at most 256, C a multiple of 8,
        * Y 32-byte aligned: the persistent kernel on pairs of SMs (thread-block clusters of two, tcgen05.mma.cta_group::2, each
        * CTA staging half of every W tile).  Same results as EGS_PATH_TENSOR; never chosen by EGS_PATH_AUTO (it measured a few
        * per cent slower); EGS_ERR_UNSUPPORTED for any other operator or shape. */
       EGS_PATH_PAIRED = 3 };
/* W memory layout relative to the contraction: CN = [E, C, N] (C rows of N), NC = [E, N, C]. */
enum { EGS_W_CN = 0, EGS_W_NC = 1 };
/* Output layout of the weight-gradient operator. */
enum { EGS_DW_GATHERED_ROWS = 0 /* out[E, FG, FD] */, EGS_DW_DIRECT_ROWS = 1 /* out[E, FD, FG] */ };

enum {
  EGS_OK = 0,
  EGS_ERR_INVALID_ARGUMENT = 1,   /* null pointer, negative size, unknown enum */
  EGS_ERR_UNSUPPORTED = 2,        /* EGS_PATH_TENSOR requested for a shape that is not eligible */
  EGS_ERR_CUDA = 3,               /* a CUDA runtime call or launch failed (see egs_last_cuda_error) */
  EGS_ERR_WORKSPACE = 4,          /* workspace missing or smaller than egs_dw_workspace_bytes says */
  EGS_ERR_TOO_LARGE = 5           /* a size exceeds an internal 32-bit or grid limit */
};

/* Bits a kernel may OR into the optional device status word (int32, caller-owned, may be NULL). */
enum {
  EGS_STATUS_INDEX_OUT_OF_RANGE = 1,  /* an Ind value outside [0,T) was met; that slot was skipped */
  EGS_STATUS_PIPELINE_TIMEOUT = 2,    /* a bounded wait inside a kernel ran out; results are invalid */
  EGS_STATUS_INTERNAL = 4             /* a kernel found its shared memory misaligned and did no work */
};

typedef struct egs_dims {
  int64_t B, T, E, K;
  int64_t C;  /* contracted feature width  (G: width of X rows;  S: width of Y rows) */
  int64_t N;  /* produced feature width    (G: width of Y rows;  S: width of Out rows) */
} egs_dims;

/* Library version (major*10000 + minor*100 + patch).  Replaces nothing in the reference. */
int egs_version(void);
const char* egs_status_string(int code);
/* Text of the last CUDA error this thread saw inside the library ("" if none). */
const char* egs_last_cuda_error(void);

/*
 * Operator G:  Y[b,e,k,n] = sum_c X[b, Ind[b,e,k], c] * W(e,c,n)
 * Replaces expert_gather_kernel + its launch wrappers:
 *   gather forward       egs/triton_kernels.py:367-392  (X=X, W=W_g [E,I,J], w_layout=EGS_W_CN, C=I, N=J)
 *   scatter backward dY  egs/triton_kernels.py:500-508  (X=dOut, W=W_s [E,J,I], w_layout=EGS_W_NC, C=I, N=J)
 * Y is fully overwritten.  Out-of-range Ind values produce a zero row and set the status bit.
 */
int egs_gather_gemm(const void* X, const void* W, const void* Ind, void* Y, const egs_dims* dims,
                    int w_layout, int dtype, int index_dtype, int precision, int path,
                    int32_t* status_word, void* cuda_stream);

/*
 * Operator S:  Out[b,t,n] (+)= sum over (e,k) with Ind[b,e,k]==t of sum_c Y[b,e,k,c] * W(e,c,n)
 * Replaces expert_scatter_kernel + its launch wrappers:
 *   scatter forward      egs/triton_kernels.py:449-474  (W=W_s [E,J,I], w_layout=EGS_W_CN, C=J, N=I)
 *   gather backward dX   egs/triton_kernels.py:416-424  (Y=dY, W=W_g [E,I,J], w_layout=EGS_W_NC, C=J, N=I)
 * zero_output != 0: Out is zero-filled first on the same stream (the reference's forward forgets to,
 * egs/triton_kernels.py:457); zero_output == 0: contributions are added to what Out holds.
 * Duplicate token ids accumulate.  The additions are atomic and their order is not fixed.
 * 16-bit tensors need egs_scatter_workspace_bytes() bytes of device scratch in workspace (contents on
 * entry do not matter; NULL is fine for float32 tensors): a planning kernel counts the contributions per
 * token row; while no row receives more than 32 the products are added straight into the 16-bit output,
 * otherwise they are summed in float32 rows of the scratch and rounded once at the end.
 */
int egs_gemm_scatter(const void* Y, const void* W, const void* Ind, void* Out, const egs_dims* dims,
                     int w_layout, int zero_output, int dtype, int index_dtype, int precision, int path,
                     void* workspace, size_t workspace_bytes, int32_t* status_word, void* cuda_stream);

/*
 * G and S with a per-expert bias fused into the epilogue: bias is [E, N] in the tensors' dtype (NULL = none).
 *   egs_gather_gemm_bias : Y[b,e,k,:] = X[b, Ind[b,e,k], :] x W(e) + bias[e]     - the `y + self.bias` of the reference's
 *                          ExpertGather.forward with its [E,1,J] parameter (egs/torch_interface.py:16-19,55), which the
 *                          reference computes with a separate elementwise kernel.
 *   egs_gemm_scatter_bias: every routed slot contributes  Y[b,e,k,:] x W(e) + bias[e]  to its token row, i.e.
 *                          Out[b,t,:] = sum over slots routed to t of (product + bias[e]).  The reference's expression
 *                          (`out + self.bias` with bias [E,1,I] against out [B,T,I], egs/torch_interface.py:71-74,111)
 *                          only broadcasts when E is 1 or B and then adds expert e's bias to batch element e; the
 *                          per-slot form is what a per-expert output bias means for routed tokens and is defined for
 *                          every shape.
 * All other arguments as in egs_gather_gemm / egs_gemm_scatter.
 */
int egs_gather_gemm_bias(const void* X, const void* W, const void* bias, const void* Ind, void* Y, const egs_dims* dims,
                         int w_layout, int dtype, int index_dtype, int precision, int path,
                         int32_t* status_word, void* cuda_stream);
int egs_gemm_scatter_bias(const void* Y, const void* W, const void* bias, const void* Ind, void* Out, const egs_dims* dims,
                          int w_layout, int zero_output, int dtype, int index_dtype, int precision, int path,
                          void* workspace, size_t workspace_bytes, int32_t* status_word, void* cuda_stream);

/* Scratch bytes egs_gemm_scatter needs (0 for float32 tensors; counters + B*T*N*4 for 16-bit ones).  No reference
 * counterpart: the reference adds atomically in the output dtype (egs/triton_kernels.py:247). */
size_t egs_scatter_workspace_bytes(int64_t B, int64_t T, int64_t N, int dtype);

/*
 * Operator D:  P[e,f,g] = sum_{b,k} Xsrc[b, Ind[b,e,k], f] * Ysrc[b,e,k,g]      (f < FG, g < FD)
 *   out_layout EGS_DW_GATHERED_ROWS : out[E, FG, FD] = P       (gather backward dW_g: Xsrc=X, Ysrc=dY)
 *   out_layout EGS_DW_DIRECT_ROWS   : out[E, FD, FG] = P^T     (scatter backward dW_s: Xsrc=dOut, Ysrc=Y)
 * Replaces expert_gather_scatter_dW_kernel + wrappers (egs/triton_kernels.py:431-439, :515-523).
 * out is fully overwritten.  workspace: egs_dw_workspace_bytes() bytes of device scratch (may be
 * NULL when that function returns 0); its contents on entry do not matter.
 */
int egs_dweight(const void* Xsrc, const void* Ysrc, const void* Ind, void* out,
                int64_t B, int64_t T, int64_t E, int64_t K, int64_t FG, int64_t FD,
                int out_layout, int dtype, int index_dtype, int precision, int path,
                void* workspace, size_t workspace_bytes, int32_t* status_word, void* cuda_stream);

/* egs_dweight for a caller that has already zero-filled a float32 `out` (the reference's wrappers do exactly that before
 * their accumulating kernel: torch.zeros_like, egs/triton_kernels.py:409 and :492): the library's own fill before a split
 * contraction is skipped, so the fill can be issued early, off the critical path.  For 16-bit tensors the promise is
 * ignored (they accumulate in the workspace) and the call equals egs_dweight. */
int egs_dweight_prezeroed(const void* Xsrc, const void* Ysrc, const void* Ind, void* out,
                          int64_t B, int64_t T, int64_t E, int64_t K, int64_t FG, int64_t FD,
                          int out_layout, int dtype, int index_dtype, int precision, int path,
                          void* workspace, size_t workspace_bytes, int32_t* status_word, void* cuda_stream);

/* Scratch bytes egs_dweight needs for these sizes (0 for float32 tensors).  No reference counterpart:
 * the reference accumulates dW with atomics directly in the output dtype (egs/triton_kernels.py:356). */
size_t egs_dw_workspace_bytes(int64_t E, int64_t FG, int64_t FD, int dtype);

/*
 * egs_dweight for callers that cannot hand over freshly allocated scratch.  (It has no counterpart in the
 * reference: there every buffer comes from torch's allocator.)  Who needs it: a host that embeds this library
 * somewhere device allocation is off limits at call time - an inference or training runtime that gives its
 * whole memory budget to its own arena at start-up and forbids cudaMalloc afterwards, a plug-in that only ever
 * sees the pointers of its inputs and outputs, or a latency-critical loop where an allocation could
 * synchronise the device or fail on a fragmented heap.  Same operator and arguments as egs_dweight, minus the
 * workspace: the float32 scratch is a 16 MiB array built into the library image (every GPU that loads the
 * library carries it until the process exits).  The entry point itself allocates nothing and frees nothing.
 *   - Limit: E*FG*FD <= egs_static_scratch_max_elements() (4 Mi elements) for 16-bit tensors; larger problems return
 *     EGS_ERR_TOO_LARGE with an explanatory egs_last_cuda_error() text and launch nothing.  float32 tensors
 *     accumulate straight into `out`, never touch the scratch and are not limited.
 *   - The first call on each device looks up the array's device address (one cudaGetSymbolAddress with
 *     that device current); make that first call outside any stream capture.
 *   - All calls share the one array, and it keeps whatever the previous call left.  Each call clears what
 *     it accumulates into, so stale contents are harmless, but two calls whose kernels may overlap on the
 *     GPU (different streams, no ordering between them) race on it: order them.
 */
int egs_dweight_static_scratch(const void* Xsrc, const void* Ysrc, const void* Ind, void* out,
                               int64_t B, int64_t T, int64_t E, int64_t K, int64_t FG, int64_t FD,
                               int out_layout, int dtype, int index_dtype, int precision, int path,
                               int32_t* status_word, void* cuda_stream);
/* Capacity of the built-in scratch in float32 elements.  No counterpart in the reference. */
size_t egs_static_scratch_max_elements(void);

/* Fused pair G -> S in ONE kernel (tensor-core path only):
 *     Mid[slot rows, N1]  = gather(Src)[slot rows, C1] x W1[e]          (overwritten; what egs_gather_gemm computes)
 *     Dst[token rows, N2] += Mid x W2[e]                                 (what egs_gemm_scatter computes)
 * The 128 x N1 tile of Mid stays on the SM between the two contractions (shared memory for float32 tensors, tensor
 * memory for 16-bit ones); it is also stored, because the backward pass and the weight gradients read it.  Both
 * weights are given in the same layout:
 *   forward  (egs/triton_kernels.py:382-390 followed by :464-472): Src = X, W1 = W_g [E,I,J], W2 = W_s [E,J,I],
 *            w_layout = EGS_W_CN, C1 = I, N1 = J, N2 = I  ->  Mid = Y, Dst = Out
 *   backward (egs/triton_kernels.py:500-508 followed by :416-424): Src = dOut, W1 = W_s [E,J,I], W2 = W_g [E,I,J],
 *            w_layout = EGS_W_NC, C1 = I, N1 = J, N2 = I  ->  Mid = dY, Dst = dX
 * The reference launches the two kernels of each pair separately; results equal those of the two separate calls
 * up to the order of the additions into Dst.  zero_output as in egs_gemm_scatter.
 * 16-bit tensors run a persistent kernel in which the tensor core works on the gather contraction of the next 128 rows
 * while the additions of the current ones drain; they need egs_scatter_workspace_bytes(B, T, N2, dtype) bytes of
 * scratch in workspace (used exactly as egs_gemm_scatter uses it); float32 tensors need none (NULL, 0).
 * Returns EGS_ERR_UNSUPPORTED when egs_fused_pair_eligible says 0: the caller then makes the two separate calls. */
int egs_gather_scatter_pair(const void* Src, const void* W1, const void* W2, const void* Ind, void* Mid, void* Dst,
                            int64_t B, int64_t T, int64_t E, int64_t K, int64_t C1, int64_t N1, int64_t N2,
                            int w_layout, int zero_output, int dtype, int index_dtype, int precision,
                            void* workspace, size_t workspace_bytes, int32_t* status_word, void* cuda_stream);
/* 1 if egs_gather_scatter_pair takes this shape on the current device (sm_100, 16-byte row pitches, tiles fit on the SM).
 * float32: N1 a multiple of 32 and <= 256, N2 within one tile (128 strict / 256 TF32).
 * 16-bit:  N1 a multiple of 16 and <= 256, C1 and N2 multiples of 8. */
int egs_fused_pair_eligible(int64_t C1, int64_t N1, int64_t N2, int w_layout, int dtype, int precision);

/*
 * Router-side index preparation.  The reference has no counterpart: its tests draw Ind with torch.randint (test_all.py:16) and
 * its scatter resolves collisions with atomics in the output dtype (egs/triton_kernels.py:235-247).
 *
 * egs_route_topk: expert-choice routing.  scores [B, T, E] float32 -> Ind [B, E, K] (any index width): for every (b, e) the K
 *   tokens with the highest score[b, :, e], best first; equal scores go to the lower token id.  K <= min(T, 1024).
 *
 * egs_index_csr: token-major CSR of Ind by counting sort (device arrays of int32, caller-owned):
 *     counts  [B*T]      slots routed to token row b*T + t
 *     offsets [B*T + 1]  exclusive prefix sums of counts
 *     entries [B*E*K]    slot ids (b*E + e)*K + k grouped by token row, ascending inside a row (reproducible)
 *     info    [4]        {heaviest row, token rows touched, 1 if an id lay outside [0,T) (such slots are left out), valid slots}
 *   scratch: egs_index_csr_scratch_bytes(B, T) bytes.  One build per step serves both scatters of the step.
 *
 * egs_index_compact: Ind (any width) -> out_dtype (EGS_I64 / EGS_I32 / EGS_I16), n = B*E*K elements; ids outside [0,T) set
 *   EGS_STATUS_INDEX_OUT_OF_RANGE in *status_word (may be NULL); T must fit the target width.
 *
 * egs_gemm_scatter_prepared: egs_gemm_scatter_bias for a caller that holds the `info` array of egs_index_csr for this Ind: the
 *   16-bit scatter's choice between direct additions and float32 rows is taken from info[0] instead of a counting pass over
 *   Ind.  csr_info = NULL makes it egs_gemm_scatter_bias.
 *
 * egs_gemm_scatter_csr: operator S evaluated token-major from the CSR: one CTA owns one token row, sums that row's
 *   contributions in CSR order in float32 and STORES the row (zeros for rows nothing is routed to; accumulate != 0 adds to
 *   what Out holds instead).  No atomics, no zero fill, no scratch, bit-reproducible.  It re-reads W[e] for every
 *   contribution, so it is the choice for small contractions or when run-to-run identical bits are required; the
 *   expert-major kernels behind egs_gemm_scatter are the fast path.  N <= 1024.
 */
int egs_route_topk(const float* scores, void* Ind, int64_t B, int64_t T, int64_t E, int64_t K, int index_dtype, void* cuda_stream);
size_t egs_index_csr_scratch_bytes(int64_t B, int64_t T);
int egs_index_csr(const void* Ind, int index_dtype, int64_t B, int64_t T, int64_t E, int64_t K, int32_t* counts, int32_t* offsets,
                  int32_t* entries, int32_t* info, void* scratch, size_t scratch_bytes, void* cuda_stream);
int egs_index_compact(const void* Ind, int index_dtype, int64_t n, int64_t T, void* out, int out_dtype, int32_t* status_word,
                      void* cuda_stream);
int egs_gemm_scatter_prepared(const void* Y, const void* W, const void* bias, const void* Ind, const int* csr_info, void* Out,
                              const egs_dims* dims, int w_layout, int zero_output, int dtype, int index_dtype, int precision,
                              int path, void* workspace, size_t workspace_bytes, int32_t* status_word, void* cuda_stream);
int egs_gemm_scatter_csr(const void* Y, const void* W, const void* bias, const int32_t* offsets, const int32_t* entries, void* Out,
                         const egs_dims* dims, int w_layout, int accumulate, int dtype, void* cuda_stream);

/* Self-test of the kernels' bounded waits (no reference counterpart).  Launches one CTA that waits, with a limit of
 * limit_cycles SM clocks (at most 2^31, about a second), on a barrier nobody completes.  The wait gives up, the kernel
 * returns normally, EGS_STATUS_PIPELINE_TIMEOUT is set in *status_word, and out2 (two ints on the device) receives
 * {1 if the wait reported failure, the CTA's abort flag}.  This is the mechanism every pipeline wait in the library uses;
 * the test shows that a wait that can never be satisfied costs its limit, not the GPU. */
int egs_selftest_wait_timeout(int32_t* status_word, int* out2, int64_t limit_cycles, void* cuda_stream);

/* 1 if EGS_PATH_AUTO would take the tcgen05 tensor-core kernels for this operator and shape, else 0.
 * op: 0 = G, 1 = S, 2 = D (for D pass C=FG, N=FD).  No reference counterpart (diagnostic). */
int egs_tensor_path_eligible(int op, const egs_dims* dims, int dtype, const void* const* pointers,
                             int n_pointers);

/* Which kernel variant EGS_PATH_AUTO runs for an operator at these sizes on the current device (no launch; base pointers are
 * assumed 16-byte aligned).  op: 0 = G, 1 = S, 2 = D (for D pass C = FG, N = FD; w_layout is ignored).  Tests use it to make
 * sure that a case reaches the variant it is meant to cover.  No reference counterpart (the reference autotunes at run time,
 * egs/triton_kernels.py:38-47). */
typedef struct egs_plan_info {
  int tensor_path;    /* 1: tcgen05 tensor-core kernels, 0: generic CUDA-core kernels (the fields below are then 0) */
  int tile_n;         /* tile width over the produced features */
  int stages;         /* depth of the shared-memory stage ring */
  int row_tiles;      /* 128-row accumulator tiles per CTA: 1 or 2 */
  int persistent;     /* G / S: 1 = the persistent warp-specialised kernel */
  int bulk_epilogue;  /* S with 16-bit tensors: direct additions go out as bulk reductions */
  int expert_fastest; /* G / S: grid order, 1 = experts vary fastest */
  int splits;         /* D: row ranges the contraction is split into */
  int rows_per_split; /* D: contraction rows per range */
} egs_plan_info;
int egs_describe_plan(int op, const egs_dims* dims, int w_layout, int dtype, int precision, egs_plan_info* out);

/* Zero-fills n bytes at p on the stream with the library's own fill kernel (what zero_output uses).
 * Replaces the torch.zeros_like calls of the reference's wrappers (egs/triton_kernels.py:408-409). */
int egs_fill_zero(void* p, size_t n_bytes, void* cuda_stream);

/* Number of kernels the library has launched in this process since load (for launch accounting). */
int64_t egs_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* EGS_B200_H_ */
