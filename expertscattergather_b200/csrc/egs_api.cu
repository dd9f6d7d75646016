// extern "C" entry points of libegs_b200.so: argument validation, path selection, launches.
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include <cuda.h>   // types of the driver API only (CUtensorMap); the entry point is looked up at run time, libcuda is not linked

#include "egs_internal.cuh"

namespace egs {

bool encode_tensor_map_16bit(TensorMap3* out, const void* base, const unsigned long long dims[3], const unsigned box[3]) {
  using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeFn encode = []() -> EncodeFn {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      return nullptr;
    return reinterpret_cast<EncodeFn>(fn);
  }();
  static_assert(sizeof(TensorMap3) == sizeof(CUtensorMap), "tensor map size");
  if (!encode || !out || !base) return false;
  const cuuint64_t gdim[3] = {dims[0], dims[1], dims[2]};
  const cuuint64_t gstride[2] = {dims[0] * 2ull, dims[0] * dims[1] * 2ull};      // bytes, dimensions 1 and 2
  const cuuint32_t bdim[3] = {box[0], box[1], box[2]};
  const cuuint32_t estride[3] = {1u, 1u, 1u};
  // CU_TENSOR_MAP_DATA_TYPE_UINT16: the loads only move bits, so one map type serves bf16 and fp16
  const CUresult rc = encode(reinterpret_cast<CUtensorMap*>(out), CU_TENSOR_MAP_DATA_TYPE_UINT16, 3u, const_cast<void*>(base), gdim,
                             gstride, bdim, estride, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return rc == CUDA_SUCCESS;
}

static std::atomic<long long> g_launches{0};
static thread_local char g_cuda_error[256] = "";

void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

namespace {

int fail_cuda(cudaError_t err, const char* where) {
  std::snprintf(g_cuda_error, sizeof(g_cuda_error), "%s: %s", where, cudaGetErrorString(err));
  return EGS_ERR_CUDA;
}

bool valid_dtype(int d) { return d == EGS_F32 || d == EGS_F16 || d == EGS_BF16; }
bool valid_index(int d) { return d == EGS_I16 || d == EGS_I32 || d == EGS_I64; }
int elem_size(int d) { return d == EGS_F32 ? 4 : 2; }
bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
constexpr long long kInt32Max = 2147483647LL;
// 16-bit scatter adds directly into the output while no token row receives more contributions than this.
constexpr int kDirect16Limit = 32;
// Longest contraction strict float32 runs on the tensor cores under EGS_PATH_AUTO (see run_rowgemm).
constexpr long long kStrictMaxContraction = 512;

bool device_is_sm100() {
  static thread_local int cached_dev = -1;
  static thread_local int cached_ok = 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return false;
  if (dev != cached_dev) {
    int major = 0;
    cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    cached_dev = dev;
    cached_ok = (major == 10);
  }
  return cached_ok != 0;
}

// The tensor-core kernels move rows with 16-byte copies: every row pitch must be a multiple of 16 bytes
// and every base pointer 16-byte aligned.
bool rowgemm_tensor_ok(const egs_dims& d, int dtype, const void* a, const void* w, const void* out) {
  const int es = elem_size(dtype);
  return (d.C * es) % 16 == 0 && (d.N * es) % 16 == 0 && aligned16(a) && aligned16(w) && aligned16(out);
}

int check_dims(const egs_dims* d) {
  if (!d) return EGS_ERR_INVALID_ARGUMENT;
  if (d->B < 0 || d->T < 0 || d->E < 0 || d->K < 0 || d->C < 0 || d->N < 0) return EGS_ERR_INVALID_ARGUMENT;
  if (d->B * d->T > kInt32Max || d->B * d->E * d->K > kInt32Max || d->C > (1 << 24) || d->N > (1 << 24) ||
      d->E > 65535 || d->B * d->K > kInt32Max)
    return EGS_ERR_TOO_LARGE;
  return EGS_OK;
}

// Grid order of the row kernels (see their comment).  Token rows touched: X rows for G, the (float32) rows added to for S.
int pick_expert_fastest(const egs_dims& d, bool scatter, int dtype) {
  const double act_bytes = static_cast<double>(d.B) * d.T * (scatter ? d.N * 4.0 : d.C * static_cast<double>(elem_size(dtype)));
  const double w_bytes = static_cast<double>(d.E) * d.C * d.N * elem_size(dtype);
  return (act_bytes > 96e6 && w_bytes < 64e6 && (d.B * d.K + 127) / 128 <= 65535) ? 1 : 0;
}

int run_rowgemm(bool scatter, const void* A, const void* W, const void* bias, const void* Ind, void* Out, const egs_dims* dims,
                int w_layout, int zero_output, int dtype, int index_dtype, int precision, int path, void* workspace,
                size_t workspace_bytes, int32_t* status, void* stream, const int* csr_info = nullptr) {
  if (int rc = check_dims(dims)) return rc;
  if (!valid_dtype(dtype) || !valid_index(index_dtype) || (w_layout != EGS_W_CN && w_layout != EGS_W_NC) ||
      (precision != EGS_PREC_STRICT && precision != EGS_PREC_TF32) ||
      (path != EGS_PATH_AUTO && path != EGS_PATH_GENERIC && path != EGS_PATH_TENSOR && path != EGS_PATH_PAIRED))
    return EGS_ERR_INVALID_ARGUMENT;
  if (path == EGS_PATH_PAIRED && (scatter || dtype == EGS_F32)) return EGS_ERR_UNSUPPORTED;
  const egs_dims& d = *dims;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const long long out_rows = scatter ? d.B * d.T : d.B * d.E * d.K;
  const size_t out_bytes = static_cast<size_t>(out_rows) * d.N * elem_size(dtype);
  if (out_bytes == 0) return EGS_OK;
  if (!Out) return EGS_ERR_INVALID_ARGUMENT;
  const bool no_work = (d.B * d.E * d.K == 0);
  if (!no_work && (!A || !W || !Ind) && d.C > 0) return EGS_ERR_INVALID_ARGUMENT;

  // 16-bit scatter.  Workspace layout: [plan flag, 256 B][per-token counters, B*T ints][float32 rows, B*T*N].
  // Generic kernels always sum in the float32 rows; the tensor-core path lets a planning kernel decide per call
  // between those and direct 16-bit additions (see egs_generic.cu).
  const bool f32_rows = scatter && dtype != EGS_F32;
  const size_t n_out = static_cast<size_t>(out_rows) * d.N;
  float* acc = nullptr;
  int* plan = nullptr;
  const bool eligible = device_is_sm100() && rowgemm_tensor_ok(d, dtype, A, W, Out);
  if ((path == EGS_PATH_TENSOR || path == EGS_PATH_PAIRED) && !eligible) return EGS_ERR_UNSUPPORTED;
  // Strict float32 on long contractions: the tensor core's accumulator additions truncate, and the error grows with the
  // contraction length (3.3e-5 of max|ref| at C = 4096 against the 1e-5 bar).  EGS_PATH_AUTO therefore keeps strict
  // float32 on the tensor cores only up to kStrictMaxContraction and takes the FFMA kernels beyond.
  const bool strict_long = (dtype == EGS_F32 && precision == EGS_PREC_STRICT && d.C > kStrictMaxContraction);
  const bool tensor = ((path == EGS_PATH_TENSOR || path == EGS_PATH_PAIRED) || (path == EGS_PATH_AUTO && eligible && !strict_long)) && !(d.C == 0) &&
                      (bias == nullptr || aligned16(bias));
  if (path == EGS_PATH_PAIRED && !tensor) return EGS_ERR_UNSUPPORTED;
  if (f32_rows) {
    const size_t need = egs_scatter_workspace_bytes(d.B, d.T, d.N, dtype);
    if (!workspace || workspace_bytes < need || !aligned16(workspace)) return EGS_ERR_WORKSPACE;
    char* ws = static_cast<char*>(workspace);
    const size_t counter_bytes = (static_cast<size_t>(out_rows) * sizeof(int) + 255) & ~static_cast<size_t>(255);
    int* counters = reinterpret_cast<int*>(ws + 256);
    acc = reinterpret_cast<float*>(ws + 256 + counter_bytes);
    cudaError_t err;
    if (tensor && !no_work && d.C > 0) {
      plan = reinterpret_cast<int*>(ws);
      if (csr_info) {   // a CSR of this Ind has been built: its heaviest-row figure decides, no pass over Ind
        err = launch_plan_from_info(csr_info, kDirect16Limit, plan, status, st);
      } else {
        err = launch_fill_zero(ws, 256 + counter_bytes, st);
        if (err == cudaSuccess)
          err = launch_scatter_plan(Ind, index_dtype, static_cast<int>(d.B), static_cast<int>(d.T), static_cast<int>(d.E),
                                    static_cast<int>(d.K), counters, plan, kDirect16Limit, status, st);
      }
      if (err == cudaSuccess) err = launch_scatter_init(plan, acc, Out, n_out, zero_output, dtype, st);
    } else {
      err = zero_output ? launch_fill_zero(acc, n_out * sizeof(float), st) : launch_convert_to_f32(Out, acc, n_out, dtype, st);
    }
    if (err != cudaSuccess) return fail_cuda(err, "scatter scratch init");
  } else if (scatter && zero_output) {
    cudaError_t err = launch_fill_zero(Out, out_bytes, st);
    if (err != cudaSuccess) return fail_cuda(err, "fill_zero");
  }
  auto finish_rows = [&]() -> int {
    if (!f32_rows) return EGS_OK;
    cudaError_t err = plan ? launch_scatter_finish(plan, acc, Out, n_out, dtype, st)
                           : launch_convert_from_f32(acc, Out, n_out, dtype, st);
    return err == cudaSuccess ? EGS_OK : fail_cuda(err, "scatter scratch convert");
  };
  if (no_work) return finish_rows();
  if (d.C == 0 && bias == nullptr) {   // empty contraction: gather output is all zeros, scatter adds nothing
    if (!scatter) {
      cudaError_t err = launch_fill_zero(Out, out_bytes, st);
      if (err != cudaSuccess) return fail_cuda(err, "fill_zero");
    }
    return finish_rows();
  }

  RowGemmParams p{};
  p.A = A; p.W = W; p.bias = bias; p.Ind = Ind; p.Out = Out; p.acc = acc; p.plan = plan; p.status = status;
  p.B = static_cast<int>(d.B); p.T = static_cast<int>(d.T); p.E = static_cast<int>(d.E); p.K = static_cast<int>(d.K);
  p.C = static_cast<int>(d.C); p.N = static_cast<int>(d.N);
  p.M = static_cast<int>(d.B * d.K);
  p.w_layout = w_layout; p.index_dtype = index_dtype;

  cudaError_t err;
  if (tensor) {
    p.expert_fastest = pick_expert_fastest(d, scatter, dtype);
    if (path == EGS_PATH_PAIRED) {
      const size_t smem2 = configure_tensor_gather2(p);
      if (smem2 == 0) return EGS_ERR_UNSUPPORTED;
      err = launch_tensor_gather2(p, dtype, smem2, st);
    } else {
      const size_t smem = configure_tensor_rowgemm(p, scatter, dtype, precision);
      err = launch_tensor_rowgemm(p, scatter, dtype, precision, smem, st);
    }
  } else {
    err = launch_generic_rowgemm(p, scatter, dtype, st);
  }
  if (err != cudaSuccess) return fail_cuda(err, scatter ? "gemm_scatter launch" : "gather_gemm launch");
  return finish_rows();
}

}  // namespace
}  // namespace egs

using namespace egs;

extern "C" {

int egs_version(void) { return 100; }

const char* egs_status_string(int code) {
  switch (code) {
    case EGS_OK: return "ok";
    case EGS_ERR_INVALID_ARGUMENT: return "invalid argument";
    case EGS_ERR_UNSUPPORTED: return "shape or device not eligible for the requested kernel family";
    case EGS_ERR_CUDA: return "CUDA error";
    case EGS_ERR_WORKSPACE: return "workspace missing or too small";
    case EGS_ERR_TOO_LARGE: return "a size exceeds an internal limit";
    default: return "unknown status";
  }
}

const char* egs_last_cuda_error(void) { return g_cuda_error; }

int64_t egs_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int egs_gather_gemm(const void* X, const void* W, const void* Ind, void* Y, const egs_dims* dims, int w_layout,
                    int dtype, int index_dtype, int precision, int path, int32_t* status_word, void* cuda_stream) {
  return run_rowgemm(false, X, W, nullptr, Ind, Y, dims, w_layout, 0, dtype, index_dtype, precision, path, nullptr, 0,
                     status_word, cuda_stream);
}

int egs_gather_gemm_bias(const void* X, const void* W, const void* bias, const void* Ind, void* Y, const egs_dims* dims,
                         int w_layout, int dtype, int index_dtype, int precision, int path, int32_t* status_word,
                         void* cuda_stream) {
  return run_rowgemm(false, X, W, bias, Ind, Y, dims, w_layout, 0, dtype, index_dtype, precision, path, nullptr, 0,
                     status_word, cuda_stream);
}

int egs_gemm_scatter(const void* Y, const void* W, const void* Ind, void* Out, const egs_dims* dims, int w_layout,
                     int zero_output, int dtype, int index_dtype, int precision, int path, void* workspace,
                     size_t workspace_bytes, int32_t* status_word, void* cuda_stream) {
  return run_rowgemm(true, Y, W, nullptr, Ind, Out, dims, w_layout, zero_output, dtype, index_dtype, precision, path, workspace,
                     workspace_bytes, status_word, cuda_stream);
}

int egs_gemm_scatter_bias(const void* Y, const void* W, const void* bias, const void* Ind, void* Out, const egs_dims* dims,
                          int w_layout, int zero_output, int dtype, int index_dtype, int precision, int path,
                          void* workspace, size_t workspace_bytes, int32_t* status_word, void* cuda_stream) {
  return run_rowgemm(true, Y, W, bias, Ind, Out, dims, w_layout, zero_output, dtype, index_dtype, precision, path, workspace,
                     workspace_bytes, status_word, cuda_stream);
}

int egs_gemm_scatter_prepared(const void* Y, const void* W, const void* bias, const void* Ind, const int* csr_info, void* Out,
                              const egs_dims* dims, int w_layout, int zero_output, int dtype, int index_dtype, int precision,
                              int path, void* workspace, size_t workspace_bytes, int32_t* status_word, void* cuda_stream) {
  return run_rowgemm(true, Y, W, bias, Ind, Out, dims, w_layout, zero_output, dtype, index_dtype, precision, path, workspace,
                     workspace_bytes, status_word, cuda_stream, csr_info);
}

int egs_route_topk(const float* scores, void* Ind, int64_t B, int64_t T, int64_t E, int64_t K, int index_dtype, void* cuda_stream) {
  if (B < 0 || T < 0 || E < 0 || K < 0 || !valid_index(index_dtype)) return EGS_ERR_INVALID_ARGUMENT;
  if (K > T || K > 1024) return EGS_ERR_UNSUPPORTED;                 // K distinct tokens per expert; the sort buffer holds 1024
  if (index_dtype == EGS_I16 && T > 32767) return EGS_ERR_TOO_LARGE;
  if (B * E > kInt32Max || B * T * E > (1LL << 40)) return EGS_ERR_TOO_LARGE;
  if (B * E * K == 0) return EGS_OK;
  if (!scores || !Ind) return EGS_ERR_INVALID_ARGUMENT;
  cudaError_t err = launch_route_topk(scores, Ind, index_dtype, static_cast<int>(B), static_cast<int>(T), static_cast<int>(E),
                                      static_cast<int>(K), static_cast<cudaStream_t>(cuda_stream));
  return err == cudaSuccess ? EGS_OK : fail_cuda(err, "route_topk launch");
}

size_t egs_index_csr_scratch_bytes(int64_t B, int64_t T) {
  if (B <= 0 || T <= 0) return 64;
  return index_csr_scratch_ints(B * T) * sizeof(int);
}

int egs_index_csr(const void* Ind, int index_dtype, int64_t B, int64_t T, int64_t E, int64_t K, int32_t* counts, int32_t* offsets,
                  int32_t* entries, int32_t* info, void* scratch, size_t scratch_bytes, void* cuda_stream) {
  egs_dims d{B, T, E, K, 0, 0};
  if (int rc = check_dims(&d)) return rc;
  if (!valid_index(index_dtype) || !offsets || !info) return EGS_ERR_INVALID_ARGUMENT;
  if (B * T > 0 && !counts) return EGS_ERR_INVALID_ARGUMENT;
  if (B * E * K > 0 && (!Ind || !entries)) return EGS_ERR_INVALID_ARGUMENT;
  if (!scratch || scratch_bytes < egs_index_csr_scratch_bytes(B, T)) return EGS_ERR_WORKSPACE;
  cudaError_t err = launch_index_csr(Ind, index_dtype, static_cast<int>(B), static_cast<int>(T), static_cast<int>(E),
                                     static_cast<int>(K), counts, offsets, entries, info, static_cast<int*>(scratch),
                                     static_cast<cudaStream_t>(cuda_stream));
  return err == cudaSuccess ? EGS_OK : fail_cuda(err, "index_csr launch");
}

int egs_index_compact(const void* Ind, int index_dtype, int64_t n, int64_t T, void* out, int out_dtype, int32_t* status_word,
                      void* cuda_stream) {
  if (n < 0 || T < 0 || !valid_index(index_dtype) || !valid_index(out_dtype)) return EGS_ERR_INVALID_ARGUMENT;
  if (out_dtype == EGS_I16 && T > 32767) return EGS_ERR_TOO_LARGE;
  if (out_dtype == EGS_I32 && T > kInt32Max) return EGS_ERR_TOO_LARGE;
  if (n == 0) return EGS_OK;
  if (!Ind || !out) return EGS_ERR_INVALID_ARGUMENT;
  cudaError_t err = launch_compact_index(Ind, index_dtype, n, T, out, out_dtype, status_word, static_cast<cudaStream_t>(cuda_stream));
  return err == cudaSuccess ? EGS_OK : fail_cuda(err, "index_compact launch");
}

int egs_gemm_scatter_csr(const void* Y, const void* W, const void* bias, const int32_t* offsets, const int32_t* entries, void* Out,
                         const egs_dims* dims, int w_layout, int accumulate, int dtype, void* cuda_stream) {
  if (int rc = check_dims(dims)) return rc;
  if (!valid_dtype(dtype) || (w_layout != EGS_W_CN && w_layout != EGS_W_NC)) return EGS_ERR_INVALID_ARGUMENT;
  const egs_dims& d = *dims;
  if (d.B * d.T * d.N == 0) return EGS_OK;
  if (!Out || !offsets) return EGS_ERR_INVALID_ARGUMENT;
  if (d.B * d.E * d.K > 0 && (!Y || !W || !entries) && d.C > 0) return EGS_ERR_INVALID_ARGUMENT;
  if (d.N > 1024 || d.C > 12000) return EGS_ERR_UNSUPPORTED;          // 8 columns per thread; one Y row in shared memory
  cudaError_t err = launch_csr_scatter(Y, W, bias, offsets, entries, Out, d.B * d.T, static_cast<int>(d.E), static_cast<int>(d.K),
                                       static_cast<int>(d.C), static_cast<int>(d.N), w_layout, accumulate, dtype,
                                       static_cast<cudaStream_t>(cuda_stream));
  return err == cudaSuccess ? EGS_OK : fail_cuda(err, "gemm_scatter_csr launch");
}

int egs_selftest_wait_timeout(int32_t* status_word, int* out2, int64_t limit_cycles, void* cuda_stream) {
  if (!status_word || !out2 || limit_cycles < 1 || limit_cycles > (1LL << 31)) return EGS_ERR_INVALID_ARGUMENT;
  if (!device_is_sm100()) return EGS_ERR_UNSUPPORTED;
  cudaError_t err = launch_wait_timeout_selftest(status_word, out2, limit_cycles, static_cast<cudaStream_t>(cuda_stream));
  return err == cudaSuccess ? EGS_OK : fail_cuda(err, "selftest launch");
}

int egs_fused_pair_eligible(int64_t C1, int64_t N1, int64_t N2, int w_layout, int dtype, int precision) {
  if (!valid_dtype(dtype) || C1 > (1 << 24) || N1 > (1 << 24) || N2 > (1 << 24) || C1 < 0 || N1 < 0 || N2 < 0) return 0;
  if (!device_is_sm100()) return 0;
  FusedParams p{};
  p.C1 = static_cast<int>(C1); p.N1 = static_cast<int>(N1); p.N2 = static_cast<int>(N2); p.w_layout = w_layout;
  if (dtype != EGS_F32) return configure_tensor_pair16(p) != 0 ? 1 : 0;
  if (precision == EGS_PREC_STRICT && C1 > kStrictMaxContraction) return 0;     // see run_rowgemm
  return configure_tensor_fused_pair(p, precision) != 0 ? 1 : 0;
}

int egs_gather_scatter_pair(const void* Src, const void* W1, const void* W2, const void* Ind, void* Mid, void* Dst,
                            int64_t B, int64_t T, int64_t E, int64_t K, int64_t C1, int64_t N1, int64_t N2, int w_layout,
                            int zero_output, int dtype, int index_dtype, int precision, void* workspace,
                            size_t workspace_bytes, int32_t* status_word, void* cuda_stream) {
  egs_dims d1{B, T, E, K, C1, N1}, d2{B, T, E, K, N1, N2};
  if (int rc = check_dims(&d1)) return rc;
  if (int rc = check_dims(&d2)) return rc;
  if (!valid_dtype(dtype) || !valid_index(index_dtype) || (w_layout != EGS_W_CN && w_layout != EGS_W_NC) ||
      (precision != EGS_PREC_STRICT && precision != EGS_PREC_TF32))
    return EGS_ERR_INVALID_ARGUMENT;
  if (!egs_fused_pair_eligible(C1, N1, N2, w_layout, dtype, precision)) return EGS_ERR_UNSUPPORTED;
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  const size_t n_dst = static_cast<size_t>(B) * T * N2;
  const size_t dst_bytes = n_dst * elem_size(dtype);
  if (dst_bytes > 0 && !Dst) return EGS_ERR_INVALID_ARGUMENT;
  const bool no_work = (B * E * K == 0);
  if (!no_work && (!Src || !W1 || !W2 || !Ind || !Mid || !Dst)) return EGS_ERR_INVALID_ARGUMENT;
  if (!no_work && (!aligned16(Src) || !aligned16(W1) || !aligned16(W2) || !aligned16(Mid) || !aligned16(Dst)))
    return EGS_ERR_UNSUPPORTED;
  FusedParams p{};
  p.Src = Src; p.W1 = W1; p.W2 = W2; p.Ind = Ind; p.Mid = Mid; p.status = status_word;
  p.B = static_cast<int>(B); p.T = static_cast<int>(T); p.E = static_cast<int>(E); p.K = static_cast<int>(K);
  p.C1 = static_cast<int>(C1); p.N1 = static_cast<int>(N1); p.N2 = static_cast<int>(N2);
  p.M = static_cast<int>(B * K);
  p.w_layout = w_layout; p.index_dtype = index_dtype;

  if (dtype == EGS_F32) {
    if (zero_output && dst_bytes > 0) {
      cudaError_t err = launch_fill_zero(Dst, dst_bytes, st);
      if (err != cudaSuccess) return fail_cuda(err, "fill_zero");
    }
    if (no_work) return EGS_OK;
    p.Dst = static_cast<float*>(Dst);
    const size_t smem = configure_tensor_fused_pair(p, precision);
    if (smem == 0) return EGS_ERR_UNSUPPORTED;
    cudaError_t err = launch_tensor_fused_pair(p, precision, smem, st);
    if (err != cudaSuccess) return fail_cuda(err, "gather_scatter_pair launch");
    return EGS_OK;
  }

  // 16-bit tensors: the scatter half works like egs_gemm_scatter (same scratch layout, same planning step)
  if (dst_bytes == 0) return EGS_OK;
  if (no_work) {
    if (zero_output) {
      cudaError_t err = launch_fill_zero(Dst, dst_bytes, st);
      if (err != cudaSuccess) return fail_cuda(err, "fill_zero");
    }
    return EGS_OK;
  }
  const size_t need = egs_scatter_workspace_bytes(B, T, N2, dtype);
  if (!workspace || workspace_bytes < need || !aligned16(workspace)) return EGS_ERR_WORKSPACE;
  char* ws = static_cast<char*>(workspace);
  const size_t counter_bytes = (static_cast<size_t>(B) * T * sizeof(int) + 255) & ~static_cast<size_t>(255);
  int* plan = reinterpret_cast<int*>(ws);
  int* counters = reinterpret_cast<int*>(ws + 256);
  float* acc = reinterpret_cast<float*>(ws + 256 + counter_bytes);
  cudaError_t err = launch_fill_zero(ws, 256 + counter_bytes, st);
  if (err == cudaSuccess)
    err = launch_scatter_plan(Ind, index_dtype, p.B, p.T, p.E, p.K, counters, plan, kDirect16Limit, status_word, st);
  if (err == cudaSuccess) err = launch_scatter_init(plan, acc, Dst, n_dst, zero_output, dtype, st);
  if (err != cudaSuccess) return fail_cuda(err, "scatter scratch init");
  p.Dst = acc; p.Out16 = Dst; p.plan = plan;
  const double act_bytes = static_cast<double>(B) * T * N2 * 4.0;
  const double w_bytes = static_cast<double>(E) * N1 * (static_cast<double>(C1) + N2) * elem_size(dtype);
  // Row-block order: experts fastest keeps the token rows being gathered from and added to (a few batch elements at a time)
  // resident in L2 while every expert's two weight tiles stream through it; worth it when the token rows exceed L2
  // and all weights fit in it next to them.
  p.expert_fastest = (act_bytes > 96e6 && w_bytes < 100e6) ? 1 : 0;
  const size_t smem = configure_tensor_pair16(p);
  if (smem == 0) return EGS_ERR_UNSUPPORTED;
  err = launch_tensor_pair16(p, dtype, smem, st);
  if (err != cudaSuccess) return fail_cuda(err, "gather_scatter_pair launch");
  err = launch_scatter_finish(plan, acc, Dst, n_dst, dtype, st);
  return err == cudaSuccess ? EGS_OK : fail_cuda(err, "scatter scratch convert");
}

size_t egs_scatter_workspace_bytes(int64_t B, int64_t T, int64_t N, int dtype) {
  if (dtype == EGS_F32 || B <= 0 || T <= 0 || N <= 0) return 0;
  const size_t counter_bytes = (static_cast<size_t>(B) * T * sizeof(int) + 255) & ~static_cast<size_t>(255);
  return 256 + counter_bytes + static_cast<size_t>(B) * T * N * sizeof(float);
}

size_t egs_dw_workspace_bytes(int64_t E, int64_t FG, int64_t FD, int dtype) {
  if (dtype == EGS_F32 || E <= 0 || FG <= 0 || FD <= 0) return 0;
  return static_cast<size_t>(E) * FG * FD * sizeof(float);
}

// out_is_zero: the caller guarantees that a float32 `out` holds zeros on entry, so the fill before a split
// contraction (which accumulates straight into `out`) is skipped.
static int dweight_impl(const void* Xsrc, const void* Ysrc, const void* Ind, void* out, int64_t B, int64_t T, int64_t E,
                        int64_t K, int64_t FG, int64_t FD, int out_layout, int dtype, int index_dtype, int precision,
                        int path, void* workspace, size_t workspace_bytes, int32_t* status_word, void* cuda_stream,
                        bool out_is_zero) {
  egs_dims d{B, T, E, K, FG, FD};
  if (int rc = check_dims(&d)) return rc;
  if (!valid_dtype(dtype) || !valid_index(index_dtype) ||
      (out_layout != EGS_DW_GATHERED_ROWS && out_layout != EGS_DW_DIRECT_ROWS) ||
      (precision != EGS_PREC_STRICT && precision != EGS_PREC_TF32) ||
      (path != EGS_PATH_AUTO && path != EGS_PATH_GENERIC && path != EGS_PATH_TENSOR))
    return EGS_ERR_INVALID_ARGUMENT;
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  const size_t n_out = static_cast<size_t>(E) * FG * FD;
  if (n_out == 0) return EGS_OK;
  if (!out) return EGS_ERR_INVALID_ARGUMENT;
  const int es = elem_size(dtype);
  if (B * K == 0) {   // nothing to sum: the gradient is zero
    if (out_is_zero && dtype == EGS_F32) return EGS_OK;
    cudaError_t err = launch_fill_zero(out, n_out * es, st);
    return err == cudaSuccess ? EGS_OK : fail_cuda(err, "fill_zero");
  }
  if (!Xsrc || !Ysrc || !Ind) return EGS_ERR_INVALID_ARGUMENT;

  DWeightParams p{};
  p.Xsrc = Xsrc; p.Ysrc = Ysrc; p.Ind = Ind; p.out = out; p.status = status_word;
  p.B = static_cast<int>(B); p.T = static_cast<int>(T); p.E = static_cast<int>(E); p.K = static_cast<int>(K);
  p.FG = static_cast<int>(FG); p.FD = static_cast<int>(FD);
  p.M = static_cast<int>(B * K);
  p.out_layout = out_layout; p.index_dtype = index_dtype;

  const bool eligible = device_is_sm100() && (FG * es) % 16 == 0 && (FD * es) % 16 == 0 && aligned16(Xsrc) &&
                        aligned16(Ysrc) && aligned16(out) && (workspace == nullptr || aligned16(workspace));
  if (path == EGS_PATH_TENSOR && !eligible) return EGS_ERR_UNSUPPORTED;
  const bool tensor = (path == EGS_PATH_TENSOR) || (path == EGS_PATH_AUTO && eligible);

  size_t smem = 0;
  if (tensor) {
    smem = configure_tensor_dweight(p, dtype, precision);
  } else {
    // generic kernel: 64x64 tiles, contraction split so that the grid covers the SMs about twice
    const long long tiles = ((FG + 63) / 64) * ((FD + 63) / 64) * E;
    long long want = (2 * 148 + tiles - 1) / tiles;
    const long long max_splits = (p.M + 15) / 16;
    if (want > max_splits) want = max_splits;
    if (want < 1) want = 1;
    long long rows = (p.M + want - 1) / want;
    rows = (rows + 15) / 16 * 16;
    p.rows_per_split = static_cast<int>(rows);
    p.splits = static_cast<int>((p.M + rows - 1) / rows);
  }
  if (static_cast<long long>(p.E) * p.splits > 65535) return EGS_ERR_TOO_LARGE;   // grid.z limit

  cudaError_t err;
  if (p.splits > 1) {
    if (dtype == EGS_F32) {
      p.acc = static_cast<float*>(out);
    } else {
      if (!workspace || workspace_bytes < n_out * sizeof(float)) return EGS_ERR_WORKSPACE;
      p.acc = static_cast<float*>(workspace);
    }
    if (!(out_is_zero && dtype == EGS_F32)) {
      err = launch_fill_zero(p.acc, n_out * sizeof(float), st);
      if (err != cudaSuccess) return fail_cuda(err, "fill_zero");
    }
  }
  err = tensor ? launch_tensor_dweight(p, dtype, precision, smem, st) : launch_generic_dweight(p, dtype, st);
  if (err != cudaSuccess) return fail_cuda(err, "dweight launch");
  if (p.splits > 1 && dtype != EGS_F32) {
    err = launch_convert_from_f32(p.acc, out, n_out, dtype, st);
    if (err != cudaSuccess) return fail_cuda(err, "convert launch");
  }
  return EGS_OK;
}

// ------------------------------------------------------------------------------------------------
// Weight gradient without any allocation by anybody: the float32 scratch of egs_dweight lives in a
// file-scope device array.  In host code the array's name is only a stand-in for the symbol, not a device
// address, so the address is asked for once per device (with that device current) and cached.
// ------------------------------------------------------------------------------------------------
#define EGS_STATIC_SCRATCH_FLOATS (4 * 1024 * 1024)          /* 16 MiB, held by every device that loads the library */
static __device__ __align__(256) float g_static_dw_scratch[EGS_STATIC_SCRATCH_FLOATS];
static std::atomic<float*> g_static_dw_scratch_addr[64];     /* per device ordinal, filled on first use */

int egs_dweight(const void* Xsrc, const void* Ysrc, const void* Ind, void* out, int64_t B, int64_t T, int64_t E,
                int64_t K, int64_t FG, int64_t FD, int out_layout, int dtype, int index_dtype, int precision, int path,
                void* workspace, size_t workspace_bytes, int32_t* status_word, void* cuda_stream) {
  return dweight_impl(Xsrc, Ysrc, Ind, out, B, T, E, K, FG, FD, out_layout, dtype, index_dtype, precision, path, workspace,
                      workspace_bytes, status_word, cuda_stream, false);
}

int egs_dweight_prezeroed(const void* Xsrc, const void* Ysrc, const void* Ind, void* out, int64_t B, int64_t T, int64_t E,
                          int64_t K, int64_t FG, int64_t FD, int out_layout, int dtype, int index_dtype, int precision,
                          int path, void* workspace, size_t workspace_bytes, int32_t* status_word, void* cuda_stream) {
  return dweight_impl(Xsrc, Ysrc, Ind, out, B, T, E, K, FG, FD, out_layout, dtype, index_dtype, precision, path, workspace,
                      workspace_bytes, status_word, cuda_stream, true);
}

int egs_dweight_static_scratch(const void* Xsrc, const void* Ysrc, const void* Ind, void* out, int64_t B, int64_t T,
                               int64_t E, int64_t K, int64_t FG, int64_t FD, int out_layout, int dtype, int index_dtype,
                               int precision, int path, int32_t* status_word, void* cuda_stream) {
  // size check first: it needs no device.  float32 tensors accumulate straight into `out` and never touch the
  // scratch, so the limit applies to 16-bit tensors only.
  if (E < 0 || FG < 0 || FD < 0) return EGS_ERR_INVALID_ARGUMENT;
  const double elements = static_cast<double>(E) * static_cast<double>(FG) * static_cast<double>(FD);
  if (dtype != EGS_F32 && elements > static_cast<double>(EGS_STATIC_SCRATCH_FLOATS)) {
    std::snprintf(g_cuda_error, sizeof(g_cuda_error),
                  "egs_dweight_static_scratch: E*FG*FD = %.0f elements exceed the built-in scratch of %d", elements,
                  EGS_STATIC_SCRATCH_FLOATS);
    return EGS_ERR_TOO_LARGE;
  }
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return fail_cuda(err, "cudaGetDevice");
  if (dev < 0 || dev >= 64) return EGS_ERR_TOO_LARGE;
  float* scratch = g_static_dw_scratch_addr[dev].load(std::memory_order_acquire);
  if (scratch == nullptr) {                                  // set-up: first call on this device
    err = cudaGetSymbolAddress(reinterpret_cast<void**>(&scratch), g_static_dw_scratch);
    if (err != cudaSuccess) return fail_cuda(err, "cudaGetSymbolAddress(static scratch)");
    if (scratch == nullptr) {
      std::snprintf(g_cuda_error, sizeof(g_cuda_error), "cudaGetSymbolAddress(static scratch) returned a null address");
      return EGS_ERR_CUDA;
    }
    g_static_dw_scratch_addr[dev].store(scratch, std::memory_order_release);   // every thread stores the same value
  }
  // egs_dweight clears the part of the scratch it accumulates into before use and reads back only what it wrote
  return egs_dweight(Xsrc, Ysrc, Ind, out, B, T, E, K, FG, FD, out_layout, dtype, index_dtype, precision, path, scratch,
                     sizeof(float) * static_cast<size_t>(EGS_STATIC_SCRATCH_FLOATS), status_word, cuda_stream);
}

size_t egs_static_scratch_max_elements(void) { return EGS_STATIC_SCRATCH_FLOATS; }

int egs_describe_plan(int op, const egs_dims* dims, int w_layout, int dtype, int precision, egs_plan_info* out) {
  if (!out || !dims || op < 0 || op > 2 || !valid_dtype(dtype) || (w_layout != EGS_W_CN && w_layout != EGS_W_NC) ||
      (precision != EGS_PREC_STRICT && precision != EGS_PREC_TF32))
    return EGS_ERR_INVALID_ARGUMENT;
  if (int rc = check_dims(dims)) return rc;
  std::memset(out, 0, sizeof(*out));
  const egs_dims& d = *dims;
  const int es = elem_size(dtype);
  out->tensor_path = (device_is_sm100() && (d.C * es) % 16 == 0 && (d.N * es) % 16 == 0) ? 1 : 0;
  if (op != 2 && dtype == EGS_F32 && precision == EGS_PREC_STRICT && d.C > kStrictMaxContraction) out->tensor_path = 0;
  if (!out->tensor_path || d.B * d.E * d.K == 0 || d.C == 0 || d.N == 0) return EGS_OK;
  if (op == 2) {
    DWeightParams p{};
    p.B = static_cast<int>(d.B); p.T = static_cast<int>(d.T); p.E = static_cast<int>(d.E); p.K = static_cast<int>(d.K);
    p.FG = static_cast<int>(d.C); p.FD = static_cast<int>(d.N); p.M = static_cast<int>(d.B * d.K);
    configure_tensor_dweight(p, dtype, precision);
    out->tile_n = p.BN; out->stages = p.stages; out->row_tiles = p.row_tiles; out->splits = p.splits;
    out->rows_per_split = p.rows_per_split;
    return EGS_OK;
  }
  RowGemmParams p{};
  p.B = static_cast<int>(d.B); p.T = static_cast<int>(d.T); p.E = static_cast<int>(d.E); p.K = static_cast<int>(d.K);
  p.C = static_cast<int>(d.C); p.N = static_cast<int>(d.N); p.M = static_cast<int>(d.B * d.K);
  p.w_layout = w_layout;
  p.expert_fastest = pick_expert_fastest(d, op == 1, dtype);
  configure_tensor_rowgemm(p, op == 1, dtype, precision);
  out->tile_n = p.BN; out->stages = p.stages; out->row_tiles = p.row_tiles; out->persistent = p.persistent;
  out->bulk_epilogue = (p.persistent || op == 1) ? p.bulk_epilogue : 0; out->expert_fastest = p.expert_fastest;
  return EGS_OK;
}

int egs_tensor_path_eligible(int op, const egs_dims* dims, int dtype, const void* const* pointers, int n_pointers) {
  if (!dims || !valid_dtype(dtype) || op < 0 || op > 2) return 0;
  if (!device_is_sm100()) return 0;
  const int es = elem_size(dtype);
  if ((dims->C * es) % 16 != 0 || (dims->N * es) % 16 != 0) return 0;
  for (int i = 0; i < n_pointers; ++i)
    if (pointers && pointers[i] && !aligned16(pointers[i])) return 0;
  return 1;
}

int egs_fill_zero(void* p, size_t n_bytes, void* cuda_stream) {
  if (n_bytes == 0) return EGS_OK;
  if (!p) return EGS_ERR_INVALID_ARGUMENT;
  cudaError_t err = launch_fill_zero(p, n_bytes, static_cast<cudaStream_t>(cuda_stream));
  return err == cudaSuccess ? EGS_OK : fail_cuda(err, "fill_zero");
}

}  // extern "C"
