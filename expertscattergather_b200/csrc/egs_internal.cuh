// Internal declarations shared by the kernel files and the C-ABI file of libegs_b200.so.
//
// Vocabulary used across the kernels:
//   slot        one routed token slot (b, e, k); its linear id is (b*E + e)*K + k
//   token row   row b*T + t of a [B,T,F] tensor (X, Out, dX, dOut), t = Ind[slot]
//   slot row    row `slot` of a [B,E,K,F] tensor (Y, dY)
//   expert row  m in [0, B*K): the m-th slot of one expert, b = m / K, k = m % K
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/egs_b200.h"

namespace egs {

// ------------------------------------------------------------------------------------------------
// element conversion
// ------------------------------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Reads Ind[pos] for any of the three index widths.
__device__ __forceinline__ long long load_index(const void* ind, int index_dtype, long long pos) {
  if (index_dtype == EGS_I64) return static_cast<const long long*>(ind)[pos];
  if (index_dtype == EGS_I32) return static_cast<const int*>(ind)[pos];
  return static_cast<const short*>(ind)[pos];
}

// ------------------------------------------------------------------------------------------------
// parameter blocks (validated on the host: every product below fits in int32 unless typed int64)
// ------------------------------------------------------------------------------------------------
struct RowGemmParams {
  const void* A;      // G: token rows [B*T, C]      S: slot rows [B*E*K, C]
  const void* W;      // [E, C, N] (EGS_W_CN) or [E, N, C] (EGS_W_NC)
  const void* Ind;    // [B, E, K]
  void* Out;          // G: slot rows [B*E*K, N]     S: token rows [B*T, N]
  float* acc;         // S with 16-bit tensors: float32 accumulation rows [B*T, N]; otherwise unused
  const int* plan;    // S with 16-bit tensors: device flag, non-zero = accumulate in the float32 rows,
                      // zero = add directly into the 16-bit output; NULL = always the float32 rows
  const void* bias;   // optional [E, N] in the tensors' dtype: bias[e, :] is added to every produced row of expert e
                      // (G: to the stored row; S: to the row before it is added to its token row); NULL = none
  int32_t* status;    // optional device status word
  int B, T, E, K, C, N;
  int M;              // expert rows per expert = B*K
  int w_layout;
  int index_dtype;
  int BN;             // tensor path: tile width over N (multiple of 16, <= 256)
  int stages;         // tensor path: pipeline depth
  int expert_fastest; // tensor path: grid order (1: experts vary fastest, row tiles slowest)
  int row_tiles;      // tensor path: 128-row accumulator tiles per CTA (1 or 2)
  int persistent;     // tensor path: 1 = persistent warp-specialised variant
  int bulk_epilogue;  // persistent scatter: rows staged in shared memory and added with bulk asynchronous reductions
};

struct DWeightParams {
  const void* Xsrc;   // token rows [B*T, FG]  (gathered through Ind)
  const void* Ysrc;   // slot rows  [B*E*K, FD]
  const void* Ind;
  void* out;          // final output in the tensors' dtype
  float* acc;         // fp32 accumulation buffer when splits > 1 (may alias out for fp32), else unused
  int32_t* status;
  int B, T, E, K, FG, FD;
  int M;              // B*K
  int out_layout;
  int index_dtype;
  int splits;         // number of row ranges the contraction is split into
  int rows_per_split; // multiple of the stage depth
  int BN;             // tensor path: tile width over FD
  int stages;
  int row_tiles;      // tensor path: 128-feature accumulator tiles per CTA over FG (1 or 2)
};

// Fused pair G -> S (tensor path only):  Mid = gather(Src) x W1[e] is stored as slot rows AND fed, without leaving the
// SM (shared memory for float32 tensors, tensor memory for 16-bit ones), into  Dst[token rows] += Mid x W2[e].
struct FusedParams {
  const void* Src;     // token rows [B*T, C1]
  const void* W1;      // [E, C1, N1] (EGS_W_CN) or [E, N1, C1] (EGS_W_NC)
  const void* W2;      // [E, N1, N2] (EGS_W_CN) or [E, N2, N1] (EGS_W_NC)
  const void* Ind;     // [B, E, K]
  void* Mid;           // slot rows [B*E*K, N1], overwritten
  float* Dst;          // float32 token rows [B*T, N2], added to (16-bit tensors: the accumulation rows of the scratch)
  void* Out16;         // 16-bit tensors: the output token rows [B*T, N2] that direct 16-bit additions go to
  const int* plan;     // 16-bit tensors: device flag, see RowGemmParams::plan
  int32_t* status;
  int B, T, E, K, C1, N1, N2;
  int M;               // B*K
  int w_layout;        // of both weights
  int index_dtype;
  int BN1, BN2;        // MMA widths (multiples of 16)
  int stages;
  int expert_fastest;  // 16-bit kernel: order of the row blocks a CTA walks (1: experts vary fastest)
  uint32_t slot_bytes; // 16-bit kernel: bytes of one ring slot
};

// ------------------------------------------------------------------------------------------------
// launchers implemented in the kernel files; each returns a cudaError_t from the launch
// ------------------------------------------------------------------------------------------------
cudaError_t launch_generic_rowgemm(const RowGemmParams& p, bool scatter, int dtype, cudaStream_t st);
cudaError_t launch_generic_dweight(const DWeightParams& p, int dtype, cudaStream_t st);
cudaError_t launch_fill_zero(void* ptr, size_t bytes, cudaStream_t st);
cudaError_t launch_convert_from_f32(const float* src, void* dst, size_t n, int dtype, cudaStream_t st);
cudaError_t launch_convert_to_f32(const void* src, float* dst, size_t n, int dtype, cudaStream_t st);
// 16-bit scatter planning (see egs_generic.cu): counts contributions per token row and raises *plan when any
// row receives more than `limit`; the init / finish kernels then act on the float32 rows or on the 16-bit output.
cudaError_t launch_scatter_plan(const void* Ind, int index_dtype, int B, int T, int E, int K, int* counters, int* plan,
                                int limit, int32_t* status, cudaStream_t st);
cudaError_t launch_scatter_init(const int* plan, float* acc, void* out16, size_t n, int zero_output, int dtype,
                                cudaStream_t st);
cudaError_t launch_scatter_finish(const int* plan, const float* acc, void* out16, size_t n, int dtype, cudaStream_t st);

// Tensor-core (tcgen05) family.  `configure_*` fills BN/stages and returns the dynamic shared memory size.
size_t configure_tensor_rowgemm(RowGemmParams& p, bool scatter, int dtype, int precision);
size_t configure_tensor_dweight(DWeightParams& p, int dtype, int precision);
cudaError_t launch_tensor_rowgemm(const RowGemmParams& p, bool scatter, int dtype, int precision,
                                  size_t smem_bytes, cudaStream_t st);
cudaError_t launch_tensor_dweight(const DWeightParams& p, int dtype, int precision, size_t smem_bytes,
                                  cudaStream_t st);

// Fused pair: `configure` returns 0 when the shape does not fit the kernel (the caller then runs G and S).
size_t configure_tensor_fused_pair(FusedParams& p, int precision);
cudaError_t launch_tensor_fused_pair(const FusedParams& p, int precision, size_t smem_bytes, cudaStream_t st);
// Fused pair for 16-bit tensors (persistent kernel, egs_pair16.cu); same conventions.
// Operator G on pairs of SMs (egs_gather2.cu, EGS_PATH_PAIRED): fills BN / stages, returns the shared memory size or 0.
size_t configure_tensor_gather2(RowGemmParams& p);
cudaError_t launch_tensor_gather2(const RowGemmParams& p, int dtype, size_t smem_bytes, cudaStream_t st);
size_t configure_tensor_pair16(FusedParams& p);
cudaError_t launch_tensor_pair16(const FusedParams& p, int dtype, size_t smem_bytes, cudaStream_t st);

// Opaque 128-byte TMA tensor map (CUtensorMap of the driver API) and its encoder for a dense 3-D tensor of 16-bit
// elements, dims[0] innermost, 128-byte swizzle, out-of-range elements read as zero.  Returns false when the driver
// refuses the geometry (strides must be multiples of 16 bytes, box sides at most 256).
struct alignas(64) TensorMap3 {
  unsigned char bytes[128];
};
bool encode_tensor_map_16bit(TensorMap3* out, const void* base, const unsigned long long dims[3], const unsigned box[3]);

// Index preparation (egs_index.cu).  All index arrays are int32 on the device.
cudaError_t launch_route_topk(const float* scores, void* ind, int index_dtype, int B, int T, int E, int K, cudaStream_t st);
size_t index_csr_scratch_ints(long long rows);
cudaError_t launch_index_csr(const void* ind, int index_dtype, int B, int T, int E, int K, int* counts, int* offsets, int* entries,
                             int* info, int* scratch, cudaStream_t st);
cudaError_t launch_compact_index(const void* ind, int index_dtype, long long n, long long T, void* out, int out_dtype,
                                 int32_t* status, cudaStream_t st);
cudaError_t launch_csr_scatter(const void* Y, const void* W, const void* bias, const int* offsets, const int* entries, void* Out,
                               long long rows, int E, int K, int C, int N, int w_layout, int accumulate, int dtype,
                               cudaStream_t st);
// *plan = (info[0] > limit): the 16-bit scatter's choice taken from a prepared CSR instead of a pass over Ind
cudaError_t launch_plan_from_info(const int* info, int limit, int* plan, int32_t* status, cudaStream_t st);

// Bounded-wait self-test (see the kernel): out = two ints on the device.
cudaError_t launch_wait_timeout_selftest(int32_t* status, int* out, long long limit_cycles, cudaStream_t st);

void count_launch(int n = 1);

}  // namespace egs
