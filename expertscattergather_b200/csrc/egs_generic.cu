// Generic CUDA-core kernels for the three operators: any sizes, any alignment, fp32 accumulation.
// They serve shapes the tensor-core kernels do not take (row pitches that are not multiples of
// 16 bytes, e.g. the odd dimensions the reference's tests draw, test_all.py:98) and are the
// on-device cross-check for the tensor-core family.  Also here: the zero-fill and fp32->dtype
// conversion kernels.
#include "egs_internal.cuh"

namespace egs {

namespace {

constexpr int TM = 64;       // output tile rows
constexpr int TN = 64;       // output tile columns
constexpr int TK = 16;       // contraction step
constexpr int PAD = 4;
constexpr int NTHREADS = 256;  // 16 x 16 threads, 4 x 4 outputs each

// ------------------------------------------------------------------------------------------------
// G and S:  tile[m, n] = sum_c A[row_a(m), c] * W(e, c, n);   G stores it, S adds it atomically
// (operator G: egs/triton_kernels.py:48-143, operator S: :156-247 in the reference)
// ------------------------------------------------------------------------------------------------
template <typename T, bool SCATTER>
__global__ void __launch_bounds__(NTHREADS) generic_rowgemm_kernel(RowGemmParams p) {
  __shared__ float As[TK][TM + PAD];
  __shared__ float Bs[TK][TN + PAD];
  __shared__ long long row_a[TM];   // element offset of the A row, -1 when masked
  __shared__ long long row_o[TM];   // element offset of the output row, -1 when masked

  const int e = blockIdx.z;
  const int m0 = blockIdx.x * TM;
  const int n0 = blockIdx.y * TN;
  const int tid = threadIdx.x;
  const T* __restrict__ A = static_cast<const T*>(p.A);
  const T* __restrict__ W = static_cast<const T*>(p.W);
  T* __restrict__ Out = static_cast<T*>(p.Out);

  if (tid < TM) {
    const int m = m0 + tid;
    long long ra = -1, ro = -1;
    if (m < p.M) {
      const int b = m / p.K, k = m - b * p.K;
      const long long slot = (static_cast<long long>(b) * p.E + e) * p.K + k;
      const long long t = load_index(p.Ind, p.index_dtype, slot);
      if (t >= 0 && t < p.T) {
        const long long tok = static_cast<long long>(b) * p.T + t;
        ra = (SCATTER ? slot : tok) * p.C;
        ro = (SCATTER ? tok : slot) * p.N;
      } else {
        if (p.status) atomicOr(p.status, EGS_STATUS_INDEX_OUT_OF_RANGE);
        if (!SCATTER) ro = slot * p.N;   // gather: the row is still written (zeros)
      }
    }
    row_a[tid] = ra;
    row_o[tid] = ro;
  }
  __syncthreads();

  const int tx = tid & 15, ty = tid >> 4;
  float acc[4][4] = {};
  const long long wbase = static_cast<long long>(e) * p.C * p.N;

  for (int c0 = 0; c0 < p.C; c0 += TK) {
#pragma unroll
    for (int i = 0; i < (TM * TK) / NTHREADS; ++i) {
      const int idx = tid + i * NTHREADS;
      const int kk = idx & (TK - 1), m = idx >> 4;
      const long long ra = row_a[m];
      const int c = c0 + kk;
      As[kk][m] = (ra >= 0 && c < p.C) ? to_f32<T>(A[ra + c]) : 0.f;
    }
    if (p.w_layout == EGS_W_CN) {
#pragma unroll
      for (int i = 0; i < (TN * TK) / NTHREADS; ++i) {
        const int idx = tid + i * NTHREADS;
        const int n = idx & (TN - 1), kk = idx >> 6;
        const int c = c0 + kk, nn = n0 + n;
        Bs[kk][n] = (c < p.C && nn < p.N) ? to_f32<T>(W[wbase + static_cast<long long>(c) * p.N + nn]) : 0.f;
      }
    } else {
#pragma unroll
      for (int i = 0; i < (TN * TK) / NTHREADS; ++i) {
        const int idx = tid + i * NTHREADS;
        const int kk = idx & (TK - 1), n = idx >> 4;
        const int c = c0 + kk, nn = n0 + n;
        Bs[kk][n] = (c < p.C && nn < p.N) ? to_f32<T>(W[wbase + static_cast<long long>(nn) * p.C + c]) : 0.f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const long long ro = row_o[ty * 4 + i];
    if (ro < 0) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int nn = n0 + tx * 4 + j;
      if (nn >= p.N) continue;
      const float v = acc[i][j] + (p.bias ? to_f32<T>(static_cast<const T*>(p.bias)[static_cast<long long>(e) * p.N + nn]) : 0.f);
      if (SCATTER) {
        if (sizeof(T) == 2) atomicAdd(p.acc + ro + nn, v);   // 16-bit: float32 accumulation rows
        else atomicAdd(reinterpret_cast<float*>(Out) + ro + nn, v);
      } else {
        Out[ro + nn] = from_f32<T>(v);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
// D:  P[e, f, g] = sum_m Xsrc[token row(m), f] * Ysrc[slot row(m), g]
// (operator D: egs/triton_kernels.py:261-356 in the reference)
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(NTHREADS) generic_dweight_kernel(DWeightParams p) {
  __shared__ float As[TK][TM + PAD];
  __shared__ float Bs[TK][TN + PAD];
  __shared__ long long row_g[TK];
  __shared__ long long row_d[TK];

  const int e = blockIdx.z / p.splits;
  const int split = blockIdx.z - e * p.splits;
  const int f0 = blockIdx.x * TM;
  const int g0 = blockIdx.y * TN;
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const T* __restrict__ Xs = static_cast<const T*>(p.Xsrc);
  const T* __restrict__ Ys = static_cast<const T*>(p.Ysrc);

  const int m_begin = split * p.rows_per_split;
  const int m_end = min(p.M, m_begin + p.rows_per_split);
  float acc[4][4] = {};

  for (int mc = m_begin; mc < m_end; mc += TK) {
    if (tid < TK) {
      const int m = mc + tid;
      long long rg = -1, rd = -1;
      if (m < m_end) {
        const int b = m / p.K, k = m - b * p.K;
        const long long slot = (static_cast<long long>(b) * p.E + e) * p.K + k;
        const long long t = load_index(p.Ind, p.index_dtype, slot);
        if (t >= 0 && t < p.T) {
          rg = (static_cast<long long>(b) * p.T + t) * p.FG;
          rd = slot * p.FD;
        } else if (p.status) {
          atomicOr(p.status, EGS_STATUS_INDEX_OUT_OF_RANGE);
        }
      }
      row_g[tid] = rg;
      row_d[tid] = rd;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < (TM * TK) / NTHREADS; ++i) {
      const int idx = tid + i * NTHREADS;
      const int f = idx & (TM - 1), kk = idx >> 6;
      const long long rg = row_g[kk];
      As[kk][f] = (rg >= 0 && f0 + f < p.FG) ? to_f32<T>(Xs[rg + f0 + f]) : 0.f;
      const long long rd = row_d[kk];
      Bs[kk][f] = (rd >= 0 && g0 + f < p.FD) ? to_f32<T>(Ys[rd + g0 + f]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }

  T* __restrict__ out = static_cast<T*>(p.out);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int f = f0 + ty * 4 + i;
    if (f >= p.FG) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int g = g0 + tx * 4 + j;
      if (g >= p.FD) continue;
      const long long off = (p.out_layout == EGS_DW_GATHERED_ROWS)
                                ? (static_cast<long long>(e) * p.FG + f) * p.FD + g
                                : (static_cast<long long>(e) * p.FD + g) * p.FG + f;
      if (p.splits > 1) {
        atomicAdd(p.acc + off, acc[i][j]);
      } else {
        out[off] = from_f32<T>(acc[i][j]);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
// zero fill and fp32 -> dtype conversion
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) fill_zero_kernel(uint4* __restrict__ p16, size_t n16, unsigned char* tail,
                                                       size_t ntail) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  const uint4 z = make_uint4(0, 0, 0, 0);
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n16; i += stride) p16[i] = z;
  if (blockIdx.x == 0 && threadIdx.x < ntail) tail[threadIdx.x] = 0;
}

__global__ void __launch_bounds__(256) fill_zero_bytes_kernel(unsigned char* p, size_t n) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) p[i] = 0;
}

template <typename T> __device__ __forceinline__ void convert8(const float* __restrict__ src, T* __restrict__ dst);

template <typename T>
__global__ void __launch_bounds__(256) convert_from_f32_kernel(const float* __restrict__ src, T* __restrict__ dst,
                                                              size_t n) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  const size_t i0 = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const bool vec = sizeof(T) == 2 && ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15u) == 0;
  const size_t n8 = vec ? n / 8 : 0;
  for (size_t i = i0; i < n8; i += stride) convert8<T>(src + 8 * i, dst + 8 * i);
  for (size_t i = n8 * 8 + i0; i < n; i += stride) dst[i] = from_f32<T>(src[i]);
}

template <typename T>
__global__ void __launch_bounds__(256) convert_to_f32_kernel(const T* __restrict__ src, float* __restrict__ dst,
                                                            size_t n) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    dst[i] = to_f32<T>(src[i]);
}

// ---- 16-bit scatter planning -------------------------------------------------------------------
// Adding straight into a bf16/fp16 output rounds at every addition, which is accurate enough only while few
// contributions meet in one token row; summing in float32 rows and rounding once is always accurate but costs
// a float32 fill, float32 atomics on a buffer twice the size and a conversion pass.  The choice is made on the
// device, per call, from the actual indices: plan != 0 selects the float32 rows.
__global__ void __launch_bounds__(256) scatter_plan_kernel(const void* __restrict__ ind, int index_dtype, int B, int T, int E,
                                                          int K, int* __restrict__ counters, int* __restrict__ plan,
                                                          int limit) {
  const long long n = static_cast<long long>(B) * E * K;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long s = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; s < n; s += stride) {
    const long long t = load_index(ind, index_dtype, s);
    if (t < 0 || t >= T) continue;
    const long long b = s / (static_cast<long long>(E) * K);
    if (atomicAdd(counters + b * T + t, 1) + 1 > limit) *plan = 1;
  }
}

template <typename T>
__global__ void __launch_bounds__(256) scatter_init_kernel(const int* __restrict__ plan, float* __restrict__ acc,
                                                          T* __restrict__ out, size_t n, int zero_output) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  const size_t i0 = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (*plan) {   // float32 rows: zero them, or seed them with what the output holds
    if (zero_output) {
      float4* a4 = reinterpret_cast<float4*>(acc);
      const size_t n4 = n / 4;
      for (size_t i = i0; i < n4; i += stride) a4[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      for (size_t i = n4 * 4 + i0; i < n; i += stride) acc[i] = 0.f;
    } else {
      for (size_t i = i0; i < n; i += stride) acc[i] = to_f32<T>(out[i]);
    }
  } else if (zero_output) {   // direct adds: only the 16-bit output needs zeroing
    uint4* o16 = reinterpret_cast<uint4*>(out);
    const size_t n8 = n / 8;
    for (size_t i = i0; i < n8; i += stride) o16[i] = make_uint4(0, 0, 0, 0);
    for (size_t i = n8 * 8 + i0; i < n; i += stride) out[i] = from_f32<T>(0.f);
  }
}

// 8 float32 values -> 8 elements of T with vector loads and one 16-byte store (T is a 16-bit type)
template <typename T>
__device__ __forceinline__ void convert8(const float* __restrict__ src, T* __restrict__ dst) {
  const float4 a = *reinterpret_cast<const float4*>(src), b = *reinterpret_cast<const float4*>(src + 4);
  T v[8] = {from_f32<T>(a.x), from_f32<T>(a.y), from_f32<T>(a.z), from_f32<T>(a.w),
            from_f32<T>(b.x), from_f32<T>(b.y), from_f32<T>(b.z), from_f32<T>(b.w)};
  *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(v);
}

template <typename T>
__global__ void __launch_bounds__(256) scatter_finish_kernel(const int* __restrict__ plan, const float* __restrict__ acc,
                                                            T* __restrict__ out, size_t n) {
  if (!*plan) return;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  const size_t i0 = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (sizeof(T) == 2) {          // (both buffers are 16-byte aligned: checked on the host)
    const size_t n8 = n / 8;
    for (size_t i = i0; i < n8; i += stride) convert8<T>(acc + 8 * i, out + 8 * i);
    for (size_t i = n8 * 8 + i0; i < n; i += stride) out[i] = from_f32<T>(acc[i]);
  } else {
    for (size_t i = i0; i < n; i += stride) out[i] = from_f32<T>(acc[i]);
  }
}

int grid_for(size_t work_items, int per_block) {
  size_t blocks = (work_items + per_block - 1) / per_block;
  const size_t cap = 148 * 8;   // a few waves of the 148 SMs; the kernels use grid-stride loops
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return static_cast<int>(blocks);
}

}  // namespace

cudaError_t launch_generic_rowgemm(const RowGemmParams& p, bool scatter, int dtype, cudaStream_t st) {
  dim3 grid((p.M + TM - 1) / TM, (p.N + TN - 1) / TN, p.E);
  dim3 block(NTHREADS);
#define EGS_LAUNCH(TY)                                                            \
  do {                                                                            \
    if (scatter) generic_rowgemm_kernel<TY, true><<<grid, block, 0, st>>>(p);     \
    else generic_rowgemm_kernel<TY, false><<<grid, block, 0, st>>>(p);            \
  } while (0)
  if (dtype == EGS_F32) EGS_LAUNCH(float);
  else if (dtype == EGS_F16) EGS_LAUNCH(__half);
  else EGS_LAUNCH(__nv_bfloat16);
#undef EGS_LAUNCH
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_generic_dweight(const DWeightParams& p, int dtype, cudaStream_t st) {
  dim3 grid((p.FG + TM - 1) / TM, (p.FD + TN - 1) / TN, p.E * p.splits);
  dim3 block(NTHREADS);
  if (dtype == EGS_F32) generic_dweight_kernel<float><<<grid, block, 0, st>>>(p);
  else if (dtype == EGS_F16) generic_dweight_kernel<__half><<<grid, block, 0, st>>>(p);
  else generic_dweight_kernel<__nv_bfloat16><<<grid, block, 0, st>>>(p);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_fill_zero(void* ptr, size_t bytes, cudaStream_t st) {
  if (bytes == 0) return cudaSuccess;
  const uintptr_t a = reinterpret_cast<uintptr_t>(ptr);
  if (a % 16 != 0) {
    fill_zero_bytes_kernel<<<grid_for(bytes, 256), 256, 0, st>>>(static_cast<unsigned char*>(ptr), bytes);
  } else {
    const size_t n16 = bytes / 16, ntail = bytes % 16;
    fill_zero_kernel<<<grid_for(n16, 256 * 4), 256, 0, st>>>(static_cast<uint4*>(ptr), n16,
                                                            static_cast<unsigned char*>(ptr) + n16 * 16, ntail);
  }
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_convert_from_f32(const float* src, void* dst, size_t n, int dtype, cudaStream_t st) {
  if (n == 0) return cudaSuccess;
  const int grid = grid_for(n, 256 * 4);
  if (dtype == EGS_F16) convert_from_f32_kernel<__half><<<grid, 256, 0, st>>>(src, static_cast<__half*>(dst), n);
  else if (dtype == EGS_BF16)
    convert_from_f32_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(src, static_cast<__nv_bfloat16*>(dst), n);
  else return cudaErrorInvalidValue;
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_scatter_plan(const void* Ind, int index_dtype, int B, int T, int E, int K, int* counters, int* plan,
                                int limit, int32_t*, cudaStream_t st) {
  const size_t n = static_cast<size_t>(B) * E * K;
  if (n == 0) return cudaSuccess;
  scatter_plan_kernel<<<grid_for(n, 256), 256, 0, st>>>(Ind, index_dtype, B, T, E, K, counters, plan, limit);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_scatter_init(const int* plan, float* acc, void* out16, size_t n, int zero_output, int dtype,
                                cudaStream_t st) {
  if (n == 0) return cudaSuccess;
  const int grid = grid_for(n, 256 * 8);
  if (dtype == EGS_F16) scatter_init_kernel<__half><<<grid, 256, 0, st>>>(plan, acc, static_cast<__half*>(out16), n, zero_output);
  else if (dtype == EGS_BF16)
    scatter_init_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(plan, acc, static_cast<__nv_bfloat16*>(out16), n, zero_output);
  else return cudaErrorInvalidValue;
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_scatter_finish(const int* plan, const float* acc, void* out16, size_t n, int dtype, cudaStream_t st) {
  if (n == 0) return cudaSuccess;
  const int grid = grid_for(n, 256 * 4);
  if (dtype == EGS_F16) scatter_finish_kernel<__half><<<grid, 256, 0, st>>>(plan, acc, static_cast<__half*>(out16), n);
  else if (dtype == EGS_BF16)
    scatter_finish_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(plan, acc, static_cast<__nv_bfloat16*>(out16), n);
  else return cudaErrorInvalidValue;
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_convert_to_f32(const void* src, float* dst, size_t n, int dtype, cudaStream_t st) {
  if (n == 0) return cudaSuccess;
  const int grid = grid_for(n, 256 * 4);
  if (dtype == EGS_F16) convert_to_f32_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half*>(src), dst, n);
  else if (dtype == EGS_BF16)
    convert_to_f32_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(src), dst, n);
  else return cudaErrorInvalidValue;
  count_launch();
  return cudaGetLastError();
}

}  // namespace egs
