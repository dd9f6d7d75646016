// Router-side index preparation and its consumers (sm_100a build, no tensor-core code: integer and byte work).
//
// The path's index tensor Ind[B,E,K] ("for batch element b, expert e processes tokens Ind[b,e,:]", reference README.md:7)
// is produced by a router in front of the gather and consumed token-major by the scatter.  The reference has neither
// step (its tests draw Ind with torch.randint, test_all.py:16, and its scatter resolves collisions with atomics,
// egs/triton_kernels.py:235-247).  Here:
//   route_topk      expert-choice routing: Ind[b,e,:] = the K tokens with the highest score[b,:,e], best first
//                   (radix select over the order-preserving bit pattern of the scores, then a bitonic sort of the K)
//   csr_*           token-major CSR of Ind by counting sort: counts / offsets per token row (b,t) and the slot ids
//                   routed to it in ascending order; also the heaviest row, the number of rows touched and a flag for
//                   out-of-range ids.  One build per step serves both scatters of the step and the 16-bit scatter's
//                   choice between direct 16-bit additions and float32 rows.
//   compact_index   Ind -> int32 / int16 with a range check
//   csr_scatter     operator S evaluated token-major from the CSR: every token row is owned by one CTA, which sums its
//                   contributions in a fixed order and STORES the row (zeros for untouched rows): no atomics, no zero
//                   fill, bit-reproducible.  It re-reads W[e] for every contribution, so it only pays where the
//                   contraction is small; the expert-major tensor-core kernels remain the fast path.
#include "egs_internal.cuh"

namespace egs {

namespace {

// ---- order-preserving key of a float: larger float <=> larger unsigned key ----
__device__ __forceinline__ uint32_t float_key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

constexpr int kTopkThreads = 256;
constexpr int kTopkMaxK = 1024;

// One CTA per (b, e).  scores: [B, T, E] float32.  Ties are broken towards the lower token id.  NaN scores order above
// +inf (their bit pattern), i.e. they are selected first.
__global__ void __launch_bounds__(kTopkThreads) route_topk_kernel(const float* __restrict__ scores, void* __restrict__ ind,
                                                                  int index_dtype, int B, int T, int E, int K) {
  __shared__ unsigned hist[256];
  __shared__ unsigned s_prefix, s_remaining, s_count_gt, s_count_eq;
  __shared__ unsigned long long sel[kTopkMaxK];    // (key << 32) | (0xFFFFFFFF - token): descending order = best first, low token first
  const int b = blockIdx.x / E, e = blockIdx.x - b * E;
  const float* col = scores + (static_cast<long long>(b) * T) * E + e;
  const int tid = threadIdx.x;

  // radix select, most significant byte first: after the loop `prefix` is the key of the K-th best element
  unsigned prefix = 0, remaining = static_cast<unsigned>(K);
  for (int shift = 24; shift >= 0; shift -= 8) {
    hist[tid] = 0;
    __syncthreads();
    const unsigned mask = (shift == 24) ? 0u : (0xFFFFFFFFu << (shift + 8));
    for (int t = tid; t < T; t += kTopkThreads) {
      const unsigned key = float_key(col[static_cast<long long>(t) * E]);
      if ((key & mask) == (prefix & mask)) atomicAdd(&hist[(key >> shift) & 255u], 1u);
    }
    __syncthreads();
    if (tid == 0) {
      unsigned need = remaining, bin = 255;
      for (;; --bin) {                       // walk from the largest digit down until the K-th element's bin
        if (hist[bin] >= need || bin == 0) break;
        need -= hist[bin];
      }
      s_prefix = prefix | (bin << shift);
      s_remaining = need;
    }
    __syncthreads();
    prefix = s_prefix;
    remaining = s_remaining;
    __syncthreads();
  }
  // collect: every key above the threshold, plus `remaining` keys equal to it, lowest token ids first
  if (tid == 0) { s_count_gt = 0; s_count_eq = 0; }
  __syncthreads();
  const unsigned n_gt = static_cast<unsigned>(K) - remaining;
  for (int t0 = 0; t0 < T; t0 += kTopkThreads) {          // in token order, so that ties resolve deterministically
    const int t = t0 + tid;
    unsigned key = 0;
    bool gt = false, eq = false;
    if (t < T) {
      key = float_key(col[static_cast<long long>(t) * E]);
      gt = key > prefix;
      eq = key == prefix;
    }
    // rank of this thread among the `eq` threads of this pass (block-wide, by thread index)
    const unsigned ballot_eq = __ballot_sync(0xffffffffu, eq);
    __shared__ unsigned warp_eq[kTopkThreads / 32];
    if ((tid & 31) == 0) warp_eq[tid >> 5] = __popc(ballot_eq);
    __syncthreads();
    unsigned before = s_count_eq;
    for (int w = 0; w < (tid >> 5); ++w) before += warp_eq[w];
    before += __popc(ballot_eq & ((1u << (tid & 31)) - 1u));
    if (gt) {
      const unsigned pos = atomicAdd(&s_count_gt, 1u);
      sel[pos] = (static_cast<unsigned long long>(key) << 32) | (0xFFFFFFFFu - static_cast<unsigned>(t));
    } else if (eq && before < remaining) {
      sel[n_gt + before] = (static_cast<unsigned long long>(key) << 32) | (0xFFFFFFFFu - static_cast<unsigned>(t));
    }
    __syncthreads();
    if (tid == 0) {
      unsigned tot = 0;
      for (int w = 0; w < kTopkThreads / 32; ++w) tot += warp_eq[w];
      s_count_eq += tot;
    }
    __syncthreads();
  }
  // bitonic sort of the K selected (padded to a power of two with zeros, which sort last), descending
  int P = 1;
  while (P < K) P <<= 1;
  for (int i = K + tid; i < P; i += kTopkThreads) sel[i] = 0ull;
  __syncthreads();
  for (int size = 2; size <= P; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int i = tid; i < P / 2; i += kTopkThreads) {
        const int lo = 2 * i - (i & (stride - 1));
        const int hi = lo + stride;
        const bool desc = ((lo & size) == 0);
        const unsigned long long a = sel[lo], c = sel[hi];
        if ((a < c) == desc) { sel[lo] = c; sel[hi] = a; }
      }
      __syncthreads();
    }
  }
  const long long out0 = (static_cast<long long>(b) * E + e) * K;
  for (int k = tid; k < K; k += kTopkThreads) {
    const long long tok = static_cast<long long>(0xFFFFFFFFu - static_cast<unsigned>(sel[k] & 0xFFFFFFFFull));
    if (index_dtype == EGS_I64) static_cast<long long*>(ind)[out0 + k] = tok;
    else if (index_dtype == EGS_I32) static_cast<int*>(ind)[out0 + k] = static_cast<int>(tok);
    else static_cast<short*>(ind)[out0 + k] = static_cast<short>(tok);
  }
}

// ---- CSR by counting sort ----------------------------------------------------------------------------------------------
// info[0] = heaviest row, info[1] = rows touched, info[2] = 1 if an id was out of range, info[3] = valid slots
__global__ void __launch_bounds__(256) csr_count_kernel(const void* __restrict__ ind, int index_dtype, int B, int T, int E, int K,
                                                       int* __restrict__ counts, int* __restrict__ info) {
  // the four summary figures are reduced per CTA in shared memory first: one global atomic per CTA and figure
  __shared__ int s_max, s_rows, s_bad, s_valid;
  if (threadIdx.x == 0) { s_max = 0; s_rows = 0; s_bad = 0; s_valid = 0; }
  __syncthreads();
  int my_max = 0, my_rows = 0, my_valid = 0;
  const long long n = static_cast<long long>(B) * E * K;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long s = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; s < n; s += stride) {
    const long long t = load_index(ind, index_dtype, s);
    if (t < 0 || t >= T) {
      s_bad = 1;
      continue;
    }
    const long long b = s / (static_cast<long long>(E) * K);
    const int c = atomicAdd(counts + b * T + t, 1) + 1;
    my_max = max(my_max, c);
    my_rows += (c == 1);
    ++my_valid;
  }
  atomicMax(&s_max, my_max);
  atomicAdd(&s_rows, my_rows);
  atomicAdd(&s_valid, my_valid);
  __syncthreads();
  if (threadIdx.x == 0) {
    atomicMax(info + 0, s_max);
    atomicAdd(info + 1, s_rows);
    if (s_bad) info[2] = 1;
    atomicAdd(info + 3, s_valid);
  }
}

constexpr int kScanBlock = 1024;      // rows per scan block (256 threads x 4)
// phase 1: per-block exclusive scan of counts into offsets, block totals into block_sums
__global__ void __launch_bounds__(256) csr_scan_blocks_kernel(const int* __restrict__ counts, int* __restrict__ offsets,
                                                             int* __restrict__ block_sums, long long rows) {
  __shared__ int warp_tot[8];
  const long long base = static_cast<long long>(blockIdx.x) * kScanBlock + threadIdx.x * 4;
  int v[4], sum = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[i] = (base + i < rows) ? counts[base + i] : 0;
    sum += v[i];
  }
  int incl = sum;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int o = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl += o;
  }
  if (lane == 31) warp_tot[warp] = incl;
  __syncthreads();
  int wbase = 0;
  for (int w = 0; w < warp; ++w) wbase += warp_tot[w];
  int run = wbase + incl - sum;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (base + i < rows) offsets[base + i] = run;
    run += v[i];
  }
  if (threadIdx.x == 255) block_sums[blockIdx.x] = wbase + incl;
}
// phase 2: one CTA turns block_sums into exclusive prefixes (serial over chunks of 256; the number of blocks is rows/1024)
__global__ void __launch_bounds__(256) csr_scan_sums_kernel(int* __restrict__ block_sums, int nblocks, int* __restrict__ total) {
  __shared__ int warp_tot[8];
  __shared__ int carry;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int c0 = 0; c0 < nblocks; c0 += 256) {
    const int i = c0 + threadIdx.x;
    const int v = (i < nblocks) ? block_sums[i] : 0;
    int incl = v;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int o = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += o;
    }
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    int wbase = carry;
    for (int w = 0; w < warp; ++w) wbase += warp_tot[w];
    if (i < nblocks) block_sums[i] = wbase + incl - v;
    __syncthreads();
    if (threadIdx.x == 255) carry = wbase + incl;
    __syncthreads();
  }
  if (threadIdx.x == 0) *total = carry;
}
// phase 3: add the block prefixes; offsets[rows] = total
__global__ void __launch_bounds__(256) csr_scan_add_kernel(int* __restrict__ offsets, const int* __restrict__ block_sums,
                                                          const int* __restrict__ total, long long rows) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < rows) offsets[i] += block_sums[i / kScanBlock];
  if (i == rows) offsets[rows] = *total;
}
// entries: every valid slot takes the next free position of its row (cursor = a zeroed copy of counts' shape)
__global__ void __launch_bounds__(256) csr_fill_kernel(const void* __restrict__ ind, int index_dtype, int B, int T, int E, int K,
                                                      const int* __restrict__ offsets, int* __restrict__ cursor,
                                                      int* __restrict__ entries) {
  const long long n = static_cast<long long>(B) * E * K;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long s = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; s < n; s += stride) {
    const long long t = load_index(ind, index_dtype, s);
    if (t < 0 || t >= T) continue;
    const long long row = (s / (static_cast<long long>(E) * K)) * T + t;
    entries[offsets[row] + atomicAdd(cursor + row, 1)] = static_cast<int>(s);
  }
}
// the positions above depend on the order the atomics ran in: sort every row's slots ascending (rows are short; one
// thread per row, insertion sort) so that the CSR - and everything computed from it - is reproducible
__global__ void __launch_bounds__(256) csr_sort_rows_kernel(const int* __restrict__ offsets, int* __restrict__ entries, long long rows) {
  const long long r = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  const int lo = offsets[r], hi = offsets[r + 1];
  for (int i = lo + 1; i < hi; ++i) {
    const int v = entries[i];
    int j = i - 1;
    while (j >= lo && entries[j] > v) {
      entries[j + 1] = entries[j];
      --j;
    }
    entries[j + 1] = v;
  }
}

template <typename TO>
__global__ void __launch_bounds__(256) compact_index_kernel(const void* __restrict__ ind, int index_dtype, long long n, long long T,
                                                           TO* __restrict__ out, int32_t* __restrict__ status) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long s = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; s < n; s += stride) {
    const long long t = load_index(ind, index_dtype, s);
    if ((t < 0 || t >= T) && status) atomicOr(status, EGS_STATUS_INDEX_OUT_OF_RANGE);
    out[s] = static_cast<TO>(t);
  }
}

// ---- token-major scatter from the CSR -----------------------------------------------------------------------------------
// One CTA per token row; thread j owns output columns j, j + 128, ...  For every slot of the row, in CSR order:
// acc[n] += sum_c Y[slot, c] * W(e, c, n) (+ bias[e, n]).  The Y row is staged in shared memory.
constexpr int kCsrThreads = 128;
constexpr int kCsrMaxCols = 8;        // columns per thread: N <= 1024
template <typename T>
__global__ void __launch_bounds__(kCsrThreads) csr_scatter_kernel(const T* __restrict__ Y, const T* __restrict__ W,
                                                                 const T* __restrict__ bias, const int* __restrict__ offsets,
                                                                 const int* __restrict__ entries, T* __restrict__ Out, int E,
                                                                 int K, int C, int N, int w_layout, int accumulate) {
  extern __shared__ float yrow[];       // [C]
  const long long row = blockIdx.x;
  const int lo = offsets[row], hi = offsets[row + 1];
  float acc[kCsrMaxCols];
#pragma unroll
  for (int i = 0; i < kCsrMaxCols; ++i) acc[i] = 0.f;
  for (int it = lo; it < hi; ++it) {
    const int slot = entries[it];
    const int e = (slot / K) % E;
    __syncthreads();
    for (int c = threadIdx.x; c < C; c += kCsrThreads) yrow[c] = to_f32<T>(Y[static_cast<long long>(slot) * C + c]);
    __syncthreads();
    const T* We = W + static_cast<long long>(e) * C * N;
#pragma unroll
    for (int i = 0; i < kCsrMaxCols; ++i) {
      const int n = threadIdx.x + i * kCsrThreads;
      if (n >= N) break;
      float s = bias ? to_f32<T>(bias[static_cast<long long>(e) * N + n]) : 0.f;
      if (w_layout == EGS_W_CN) {
        for (int c = 0; c < C; ++c) s = fmaf(yrow[c], to_f32<T>(We[static_cast<long long>(c) * N + n]), s);
      } else {
        const T* wr = We + static_cast<long long>(n) * C;
        for (int c = 0; c < C; ++c) s = fmaf(yrow[c], to_f32<T>(wr[c]), s);
      }
      acc[i] += s;
    }
  }
#pragma unroll
  for (int i = 0; i < kCsrMaxCols; ++i) {
    const int n = threadIdx.x + i * kCsrThreads;
    if (n >= N) break;
    const long long o = row * N + n;
    Out[o] = from_f32<T>(accumulate ? to_f32<T>(Out[o]) + acc[i] : acc[i]);
  }
}

__global__ void plan_from_info_kernel(const int* __restrict__ info, int limit, int* __restrict__ plan, int32_t* status) {
  *plan = (info[0] > limit) ? 1 : 0;
  if (info[2] && status) atomicOr(status, EGS_STATUS_INDEX_OUT_OF_RANGE);
}

int grid_1d(long long items, int per_block, int cap) {
  long long blocks = (items + per_block - 1) / per_block;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return static_cast<int>(blocks);
}

}  // namespace

cudaError_t launch_route_topk(const float* scores, void* ind, int index_dtype, int B, int T, int E, int K, cudaStream_t st) {
  route_topk_kernel<<<B * E, kTopkThreads, 0, st>>>(scores, ind, index_dtype, B, T, E, K);
  count_launch();
  return cudaGetLastError();
}

size_t index_csr_scratch_ints(long long rows) { return static_cast<size_t>(rows) + static_cast<size_t>((rows + kScanBlock - 1) / kScanBlock) + 8; }

// counts [rows], offsets [rows + 1], entries [N], info [4], scratch [index_csr_scratch_ints(rows)] - all int32 on the device
cudaError_t launch_index_csr(const void* ind, int index_dtype, int B, int T, int E, int K, int* counts, int* offsets, int* entries,
                             int* info, int* scratch, cudaStream_t st) {
  const long long rows = static_cast<long long>(B) * T;
  const long long n = static_cast<long long>(B) * E * K;
  const int nblocks = static_cast<int>((rows + kScanBlock - 1) / kScanBlock);
  int* cursor = scratch;
  int* block_sums = scratch + rows;
  int* total = block_sums + nblocks;
  cudaError_t err = launch_fill_zero(counts, static_cast<size_t>(rows) * sizeof(int), st);
  if (err == cudaSuccess) err = launch_fill_zero(info, 4 * sizeof(int), st);
  if (err == cudaSuccess) err = launch_fill_zero(cursor, static_cast<size_t>(rows) * sizeof(int), st);
  if (err != cudaSuccess) return err;
  if (n > 0) csr_count_kernel<<<grid_1d(n, 256, 148 * 8), 256, 0, st>>>(ind, index_dtype, B, T, E, K, counts, info);
  if (rows > 0) {
    csr_scan_blocks_kernel<<<nblocks, 256, 0, st>>>(counts, offsets, block_sums, rows);
    csr_scan_sums_kernel<<<1, 256, 0, st>>>(block_sums, nblocks, total);
    csr_scan_add_kernel<<<static_cast<int>((rows + 1 + 255) / 256), 256, 0, st>>>(offsets, block_sums, total, rows);
  } else {
    err = launch_fill_zero(offsets, sizeof(int), st);
    if (err != cudaSuccess) return err;
  }
  if (n > 0) {
    csr_fill_kernel<<<grid_1d(n, 256, 148 * 8), 256, 0, st>>>(ind, index_dtype, B, T, E, K, offsets, cursor, entries);
    csr_sort_rows_kernel<<<static_cast<int>((rows + 255) / 256), 256, 0, st>>>(offsets, entries, rows);
  }
  count_launch(n > 0 ? 6 : 3);
  return cudaGetLastError();
}

cudaError_t launch_plan_from_info(const int* info, int limit, int* plan, int32_t* status, cudaStream_t st) {
  plan_from_info_kernel<<<1, 1, 0, st>>>(info, limit, plan, status);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_compact_index(const void* ind, int index_dtype, long long n, long long T, void* out, int out_dtype,
                                 int32_t* status, cudaStream_t st) {
  if (n == 0) return cudaSuccess;
  const int grid = grid_1d(n, 256, 148 * 8);
  if (out_dtype == EGS_I64) compact_index_kernel<long long><<<grid, 256, 0, st>>>(ind, index_dtype, n, T, static_cast<long long*>(out), status);
  else if (out_dtype == EGS_I32) compact_index_kernel<int><<<grid, 256, 0, st>>>(ind, index_dtype, n, T, static_cast<int*>(out), status);
  else compact_index_kernel<short><<<grid, 256, 0, st>>>(ind, index_dtype, n, T, static_cast<short*>(out), status);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_csr_scatter(const void* Y, const void* W, const void* bias, const int* offsets, const int* entries, void* Out,
                               long long rows, int E, int K, int C, int N, int w_layout, int accumulate, int dtype,
                               cudaStream_t st) {
  if (rows == 0 || N == 0) return cudaSuccess;
  const size_t smem = static_cast<size_t>(C) * sizeof(float);
  const unsigned grid = static_cast<unsigned>(rows);
#define EGS_CSR(TY)                                                                                                       \
  csr_scatter_kernel<TY><<<grid, kCsrThreads, smem, st>>>(static_cast<const TY*>(Y), static_cast<const TY*>(W),           \
                                                        static_cast<const TY*>(bias), offsets, entries, static_cast<TY*>(Out), \
                                                        E, K, C, N, w_layout, accumulate)
  if (dtype == EGS_F32) EGS_CSR(float);
  else if (dtype == EGS_F16) EGS_CSR(__half);
  else EGS_CSR(__nv_bfloat16);
#undef EGS_CSR
  count_launch();
  return cudaGetLastError();
}

}  // namespace egs
