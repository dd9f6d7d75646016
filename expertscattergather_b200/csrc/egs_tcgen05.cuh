// Device-side building blocks of the tcgen05 / TMEM kernels (sm_100a): PTX wrappers, bounded mbarrier waits,
// shared-memory and instruction descriptors, the swizzled tile addressing and the epilogue helpers.
// Included by every kernel file of the tensor-core family; everything here has internal linkage.
//
// Shared-memory tile format (one format for every operand): rows of 128-byte segments.  Element
// (row r, 16-byte chunk c of the row) lives at
//     base + (c / 8) * seg_stride + (r / 8) * 1024 + (r % 8) * 128 + ((c % 8) ^ (r % 8)) * 16
// i.e. 8-row x 128-byte atoms with the hardware's 128B XOR swizzle, atoms of one segment column stacked
// 1024 bytes apart, segment columns seg_stride = rows*128 bytes apart.  Read with a K-major descriptor
// (rows = M or N index, SBO = 1024) the row is a contraction-contiguous operand; read with an MN-major
// descriptor (rows = contraction index, LBO = seg_stride, SBO = 1024) the same bytes are a transposed
// operand.  The tensor core reads MN-major 32-bit (TF32) operands only in the variant of this format whose
// XOR acts on 32-byte pairs with the row index modulo 4 (atoms of 4 rows; SBO = 512).
#pragma once

#include "egs_internal.cuh"

namespace egs {
namespace {

constexpr int kProducerWarps = 8;
constexpr int kProducerThreads = kProducerWarps * 32;
constexpr int kThreads = kProducerThreads + 32;
constexpr int kTileM = 128;
constexpr int kMaxStages = 8;
constexpr uint32_t kHeaderBytes = 3072;       // row kernel: barriers + two row tables
constexpr uint32_t kHeaderBytesD = 1024;      // weight-gradient kernel: barriers only (the row tables are unused)
constexpr long long kWaitLimitCycles = 1LL << 31;   // about a second at B200 clocks

// Upper bound, in nanoseconds, on how long one mbarrier.try_wait keeps the thread suspended before it returns
// "not yet" (the thread is resumed at once when the phase completes).  Long suspensions keep waiting warps from
// taking issue slots away from the warps that have work.
constexpr uint32_t kTryWaitSuspendNs = 1000000u;

constexpr int kMaxRowsPerSplit = 8192;   // operator D: contraction rows one CTA may own (row table in smem, 32 KB)

struct __align__(16) SmemHeader {
  unsigned long long full[kMaxStages];
  unsigned long long empty[kMaxStages];
  unsigned long long done;
  unsigned long long drain;   // spare barrier: the exit path waits on it for MMAs still in flight after an abort
  uint32_t tmem_base;
  uint32_t abort_flag;
  int row_a[2 * kTileM];   // rowgemm: source row index per CTA row (-1 = masked)
  int row_o[2 * kTileM];   // rowgemm: destination row index per CTA row (-1 = masked)
};
static_assert(sizeof(SmemHeader) <= kHeaderBytes, "header does not fit");

// ------------------------------------------------------------------------------------------------
// PTX wrappers
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async16_full(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
// Hardware arrive on an mbarrier once all cp.async copies this thread has issued so far have landed.
__device__ __forceinline__ void cp_async_mbar_arrive_noinc(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_pending(int n) {
  switch (n) {
    case 0: asm volatile("cp.async.wait_group 0;" ::: "memory"); break;
    case 1: asm volatile("cp.async.wait_group 1;" ::: "memory"); break;
    case 2: asm volatile("cp.async.wait_group 2;" ::: "memory"); break;
    case 3: asm volatile("cp.async.wait_group 3;" ::: "memory"); break;
    case 4: asm volatile("cp.async.wait_group 4;" ::: "memory"); break;
    case 5: asm volatile("cp.async.wait_group 5;" ::: "memory"); break;
    default: asm volatile("cp.async.wait_group 6;" ::: "memory"); break;
  }
}
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(bar) : "memory");
}
// Announces `bytes` of asynchronous (TMA) traffic that will complete on the barrier and arrives on it once.
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}" ::"r"(bar), "r"(bytes) : "memory");
}
// TMA tile load into this CTA's own shared memory: box of a 3-D tensor map, bytes counted on `bar`.
// The innermost coordinate times the element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_3d(uint32_t dst_smem, const void* tensor_map, int x, int y, int z, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst_smem),
      "l"(tensor_map), "r"(x), "r"(y), "r"(z), "r"(bar)
      : "memory");
}
__device__ __forceinline__ uint32_t mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(kTryWaitSuspendNs)
      : "memory");
  return ok;
}
// Bounded wait.  Returns false when the CTA is aborting (this or another thread ran out of time).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag,
                                          int32_t* status, long long limit_cycles = kWaitLimitCycles) {
  if (mbar_try(bar, parity)) return true;
  const long long t0 = clock64();
  uint32_t spins = 0;
  for (;;) {
    if (mbar_try(bar, parity)) return true;
    if (((++spins) & 63u) == 0u) {
      if (*abort_flag) return false;
      if (clock64() - t0 > limit_cycles) {
        *abort_flag = 1u;
        if (status) atomicOr(status, EGS_STATUS_PIPELINE_TIMEOUT);
        return false;
      }
    }
  }
}

// One lane polls, the warp shares the outcome (keeps 31 lanes per warp off the barrier word).
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag,
                                               int32_t* status, int lane) {
  uint32_t ok = 1u;
  if (lane == 0) ok = mbar_wait(bar, parity, abort_flag, status) ? 1u : 0u;
  return __shfl_sync(0xffffffffu, ok, 0) != 0u;
}

__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
template <bool TF32>
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  if (TF32) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
// tcgen05.mma with the A operand in tensor memory (K-major only): lane = row, every 32-bit column holds two
// consecutive 16-bit contraction elements (low half first); one instruction consumes 8 columns (16 elements).
__device__ __forceinline__ void umma_ts_f16(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(tmem_d),
      "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Straight-line groups of tcgen05.mma (kind::f16) with the descriptor arithmetic inside the PTX block: the issuing lane
// runs alone, so every instruction it executes costs a full issue latency and loops around single MMAs starve the
// tensor core.  The start-address field of a shared-memory descriptor is its low 14 bits (16-byte units), so advancing
// an operand is a 64-bit add of a small number.
//   four contraction steps, both operands in shared memory; A advances by a_adv, B by b_adv per step
__device__ __forceinline__ void umma_ss_f16_x4(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t a_adv, uint32_t b_adv,
                                               uint32_t idesc, uint32_t accumulate_first) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t.reg .b64 aa, bb, a, b;\n\t"
      "setp.ne.b32 p, %6, 0;\n\tsetp.eq.b32 q, 0, 0;\n\t"
      "cvt.u64.u32 aa, %3;\n\tcvt.u64.u32 bb, %4;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %5, p;\n\t"
      "add.u64 a, %1, aa;\n\tadd.u64 b, %2, bb;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %5, q;\n\t"
      "add.u64 a, a, aa;\n\tadd.u64 b, b, bb;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %5, q;\n\t"
      "add.u64 a, a, aa;\n\tadd.u64 b, b, bb;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %5, q;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(a_adv), "r"(b_adv), "r"(idesc), "r"(accumulate_first)
      : "memory");
}
//   eight contraction steps with A in tensor memory (8 columns per step); B advances by b_adv per step and by another
//   b_jump after the fourth (the next 128-byte segment of a K-major tile)
__device__ __forceinline__ void umma_ts_f16_x8(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t b_adv, uint32_t b_jump,
                                               uint32_t idesc, uint32_t accumulate_first) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t.reg .b64 bb, bj, b;\n\t.reg .b32 a;\n\t"
      "setp.ne.b32 p, %6, 0;\n\tsetp.eq.b32 q, 0, 0;\n\t"
      "cvt.u64.u32 bb, %3;\n\tcvt.u64.u32 bj, %4;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %5, p;\n\t"
      "add.u32 a, %1, 8;\n\tadd.u64 b, %2, bb;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %5, q;\n\t"
      "add.u32 a, a, 8;\n\tadd.u64 b, b, bb;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %5, q;\n\t"
      "add.u32 a, a, 8;\n\tadd.u64 b, b, bb;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %5, q;\n\t"
      "add.u32 a, a, 8;\n\tadd.u64 b, b, bb;\n\tadd.u64 b, b, bj;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %5, q;\n\t"
      "add.u32 a, a, 8;\n\tadd.u64 b, b, bb;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %5, q;\n\t"
      "add.u32 a, a, 8;\n\tadd.u64 b, b, bb;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %5, q;\n\t"
      "add.u32 a, a, 8;\n\tadd.u64 b, b, bb;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %5, q;\n\t}" ::"r"(tmem_d),
      "r"(tmem_a), "l"(bdesc), "r"(b_adv), "r"(b_jump), "r"(idesc), "r"(accumulate_first)
      : "memory");
}
// Writes 16 consecutive 32-bit columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// 16 consecutive fp32 accumulator columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
// 32 consecutive fp32 accumulator columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor, sm_100 version field set.  layout_type 2 = 128-byte swizzle (16-byte
// granules, 8-row atoms); 1 = 128-byte swizzle with 32-byte granules and 4-row atoms, the only layout the
// tensor core accepts for MN-major (transposed) 32-bit operands.
constexpr uint32_t kSwizzle128 = 2, kSwizzle128Base32 = 1;
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                                   uint32_t layout_type = kSwizzle128) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr >> 4) & 0x3FFFu);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= static_cast<uint64_t>(1) << 46;   // descriptor version of this architecture
  d |= static_cast<uint64_t>(layout_type) << 61;
  return d;
}
// Instruction descriptor: fp32 accumulator, A and B of one format (0 f16, 1 bf16, 2 tf32).
__device__ __forceinline__ uint32_t make_idesc(uint32_t fmt, uint32_t a_mn_major, uint32_t b_mn_major, uint32_t m,
                                               uint32_t n) {
  return (1u << 4) | (fmt << 7) | (fmt << 10) | (a_mn_major << 15) | (b_mn_major << 16) | ((n >> 3) << 17) |
         ((m >> 4) << 24);
}

// Address of (row r, 16-byte chunk c) inside a tile in the format described at the top of the file.
// BASE32 selects the 32-byte-granule swizzle: rows stay 128 bytes apart, but the XOR acts on the 32-byte
// pair index with the row index modulo 4 (atoms of 4 rows, 512 bytes).
template <bool BASE32>
__device__ __forceinline__ uint32_t tile_addr(uint32_t base, uint32_t seg_stride, int r, int c) {
  const uint32_t row = base + static_cast<uint32_t>(c >> 3) * seg_stride + static_cast<uint32_t>(r) * 128u;
  if (BASE32) return row + (static_cast<uint32_t>(((c & 7) >> 1) ^ (r & 3)) << 5) + (static_cast<uint32_t>(c & 1) << 4);
  return row + (static_cast<uint32_t>((c & 7) ^ (r & 7)) << 4);
}

// In-place hi/lo split of one 16-byte chunk of float32 values (strict mode).
__device__ __forceinline__ void split_chunk(uint32_t addr, uint32_t lo_offset) {
  uint32_t v[4], lo[4];
  asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]) : "r"(addr) : "memory");
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t hi = v[i] & 0xFFFFE000u;
    const float rem = __uint_as_float(v[i]) - __uint_as_float(hi);
    lo[i] = (__float_as_uint(rem) + 0x1000u) & 0xFFFFE000u;   // round to tf32 (nearest, ties away) with integer ops
    v[i] = hi;
  }
  asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]) : "memory");
  asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(addr + lo_offset), "r"(lo[0]), "r"(lo[1]), "r"(lo[2]), "r"(lo[3])
               : "memory");
}

template <typename T> struct Elem;
template <> struct Elem<float> { static constexpr uint32_t fmt = 2; static constexpr bool tf32 = true; };
template <> struct Elem<__half> { static constexpr uint32_t fmt = 0; static constexpr bool tf32 = false; };
template <> struct Elem<__nv_bfloat16> { static constexpr uint32_t fmt = 1; static constexpr bool tf32 = false; };


// ---- epilogue helpers ----
__device__ __forceinline__ uint32_t pack2(__half*, uint32_t a, uint32_t b) {
  const __half2 h = __floats2half2_rn(__uint_as_float(a), __uint_as_float(b));
  return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t pack2(__nv_bfloat16*, uint32_t a, uint32_t b) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(a), __uint_as_float(b));
  return *reinterpret_cast<const uint32_t*>(&h);
}
// Warp-level transpose of a 32-row x 32-column fp32 accumulator block through a 4 KB shared-memory tile.
// In tensor memory one thread owns one row, which would make every global access of a warp touch 32
// different rows (16 bytes each).  After the transpose 8 lanes cover 128 contiguous bytes of one row, 4 rows
// per instruction; for red.global.add that pattern measured ~3x the throughput of the row-per-thread one.
//   emit(row_in_block, first_column, x0, x1, x2, x3) is called 8 times per lane.
template <class Emit>
__device__ __forceinline__ void warp_block_emit(uint32_t taddr, uint32_t tile, int lane, bool have_acc, Emit&& emit) {
  uint32_t v[32];
  if (have_acc) {
    tmem_ld32(taddr, v);
    tmem_ld_wait();
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = 0u;
  }
#pragma unroll
  for (int j = 0; j < 8; ++j)
    asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(tile + lane * 128u + (static_cast<uint32_t>(j ^ (lane & 7)) << 4)),
                 "r"(v[4 * j]), "r"(v[4 * j + 1]), "r"(v[4 * j + 2]), "r"(v[4 * j + 3])
                 : "memory");
  __syncwarp();
  const int j = lane & 7;
  uint32_t x[8][4];
#pragma unroll
  for (int it = 0; it < 8; ++it) {      // all reads first, so that their latencies overlap
    const int row = it * 4 + (lane >> 3);
    asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(x[it][0]), "=r"(x[it][1]), "=r"(x[it][2]), "=r"(x[it][3])
                 : "r"(tile + row * 128u + (static_cast<uint32_t>(j ^ (row & 7)) << 4))
                 : "memory");
  }
  __syncwarp();                         // the tile may be overwritten from here on
#pragma unroll
  for (int it = 0; it < 8; ++it) emit(it * 4 + (lane >> 3), j * 4, x[it][0], x[it][1], x[it][2], x[it][3]);
}
// Same transpose for a 32-row x 64-column block (8 KB tile): every lane ends up with 8 consecutive columns of
// one row, so 8 lanes cover 64 columns - 128 contiguous bytes of a 16-bit row per instruction.
//   emit(row_in_block, first_column, x[8]) is called 8 times per lane.
template <class Emit>
__device__ __forceinline__ void warp_block_emit64(uint32_t taddr, uint32_t tile, int lane, Emit&& emit) {
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    uint32_t v[32];
    tmem_ld32(taddr + h * 32, v);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < 8; ++j)
      asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(tile + lane * 256u + (static_cast<uint32_t>((h * 8 + j) ^ (lane & 7)) << 4)),
                   "r"(v[4 * j]), "r"(v[4 * j + 1]), "r"(v[4 * j + 2]), "r"(v[4 * j + 3])
                   : "memory");
  }
  __syncwarp();
  const int j = lane & 7;
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int row = it * 4 + (lane >> 3);
    uint32_t x[8];
#pragma unroll
    for (int q = 0; q < 2; ++q)
      asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];"
                   : "=r"(x[4 * q]), "=r"(x[4 * q + 1]), "=r"(x[4 * q + 2]), "=r"(x[4 * q + 3])
                   : "r"(tile + row * 256u + (static_cast<uint32_t>((2 * j + q) ^ (row & 7)) << 4))
                   : "memory");
    emit(row, j * 8, x);
  }
  __syncwarp();
}
__device__ __forceinline__ void red8(__nv_bfloat16* dst, const uint32_t (&x)[8]) {
  asm volatile("red.global.add.noftz.v4.bf16x2 [%0], {%1,%2,%3,%4};" ::"l"(dst), "r"(pack2(dst, x[0], x[1])),
               "r"(pack2(dst, x[2], x[3])), "r"(pack2(dst, x[4], x[5])), "r"(pack2(dst, x[6], x[7]))
               : "memory");
}
__device__ __forceinline__ void red8(__half* dst, const uint32_t (&x)[8]) {
  asm volatile("red.global.add.noftz.v4.f16x2 [%0], {%1,%2,%3,%4};" ::"l"(dst), "r"(pack2(dst, x[0], x[1])),
               "r"(pack2(dst, x[2], x[3])), "r"(pack2(dst, x[4], x[5])), "r"(pack2(dst, x[6], x[7]))
               : "memory");
}
__device__ __forceinline__ void red8(float*, const uint32_t (&)[8]) {}   // never taken: direct adds are 16-bit only
// Bulk asynchronous reduction: adds `bytes` (multiple of 16) of elements staged in shared memory to global memory.
// The copy engine reads the shared memory after the instruction has issued: the staging buffer may be rewritten
// only after bulk_wait_read, and the issuing thread's own writes need fence.proxy.async before the instruction.
__device__ __forceinline__ void bulk_reduce_add(__nv_bfloat16* dst, uint32_t src_smem, uint32_t bytes) {
  asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.noftz.bf16 [%0], [%1], %2;" ::"l"(dst), "r"(src_smem),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_reduce_add(__half* dst, uint32_t src_smem, uint32_t bytes) {
  asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.noftz.f16 [%0], [%1], %2;" ::"l"(dst), "r"(src_smem),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
constexpr uint32_t kBulkRowPitch = 144;                  // 128 staged bytes per row + 16: conflict-free 16-byte stores
constexpr uint32_t kBulkBufBytes = 32 * kBulkRowPitch;   // one 32-row staging buffer
__device__ __forceinline__ void red4(float* dst, uint32_t x0, uint32_t x1, uint32_t x2, uint32_t x3) {
  asm volatile("red.global.add.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(dst), "f"(__uint_as_float(x0)), "f"(__uint_as_float(x1)),
               "f"(__uint_as_float(x2)), "f"(__uint_as_float(x3))
               : "memory");
}
__device__ __forceinline__ void red4(__nv_bfloat16* dst, uint32_t x0, uint32_t x1, uint32_t x2, uint32_t x3) {
  asm volatile("red.global.add.noftz.v2.bf16x2 [%0], {%1,%2};" ::"l"(dst), "r"(pack2(dst, x0, x1)), "r"(pack2(dst, x2, x3)) : "memory");
}
__device__ __forceinline__ void red4(__half* dst, uint32_t x0, uint32_t x1, uint32_t x2, uint32_t x3) {
  asm volatile("red.global.add.noftz.v2.f16x2 [%0], {%1,%2};" ::"l"(dst), "r"(pack2(dst, x0, x1)), "r"(pack2(dst, x2, x3)) : "memory");
}
__device__ __forceinline__ void store4(float* dst, uint32_t x0, uint32_t x1, uint32_t x2, uint32_t x3) {
  *reinterpret_cast<uint4*>(dst) = make_uint4(x0, x1, x2, x3);
}
template <typename T>
__device__ __forceinline__ void store4(T* dst, uint32_t x0, uint32_t x1, uint32_t x2, uint32_t x3) {
  *reinterpret_cast<uint2*>(dst) = make_uint2(pack2(dst, x0, x1), pack2(dst, x2, x3));
}

// Adds bias[0..3] (elements of type T, 4 consecutive columns) to four accumulator values held as float bits.
template <typename T>
__device__ __forceinline__ void add_bias4(const T* bias, uint32_t& x0, uint32_t& x1, uint32_t& x2, uint32_t& x3) {
  x0 = __float_as_uint(__uint_as_float(x0) + to_f32<T>(bias[0]));
  x1 = __float_as_uint(__uint_as_float(x1) + to_f32<T>(bias[1]));
  x2 = __float_as_uint(__uint_as_float(x2) + to_f32<T>(bias[2]));
  x3 = __float_as_uint(__uint_as_float(x3) + to_f32<T>(bias[3]));
}

__device__ __forceinline__ uint32_t tmem_cols_for(int bn) {
  uint32_t c = 32;
  while (c < static_cast<uint32_t>(bn)) c <<= 1;
  return c;
}

// The dynamic shared memory is declared 1024-byte aligned (the swizzle atoms need it).  Should a launch ever
// hand out a differently aligned base, the CTA refuses to work and reports EGS_STATUS_INTERNAL.
__device__ __forceinline__ bool smem_misaligned(const void* raw) { return (smem_u32(raw) & 1023u) != 0u; }

// Common exit of the warp that owns the tensor-memory allocation (all 32 lanes call it, after the CTA-wide barrier of
// the exit path).  After an abort tcgen05.mma operations may still be in flight: one lane commits them to the spare
// barrier `drain_bar` (initialised with count 1, never used otherwise) and waits for it, again with a limit, before
// the columns are released; if even that wait runs out the columns stay allocated until the CTA exits rather than
// being released under running MMAs.
__device__ __forceinline__ void tmem_release(uint32_t tmem_base, uint32_t ncols, uint32_t drain_bar, volatile uint32_t* abort_flag,
                                             int lane) {
  uint32_t safe = 1u;
  if (*abort_flag) {
    if (lane == 0) {
      uint32_t ignore_abort = 0u;      // the CTA's abort flag is already up: this wait must not return early on it
      umma_commit(drain_bar);
      safe = mbar_wait(drain_bar, 0u, &ignore_abort, nullptr) ? 1u : 0u;
    }
    safe = __shfl_sync(0xffffffffu, safe, 0);
  }
  if (safe) {
    tc_fence_after();
    tmem_dealloc(tmem_base, ncols);
  }
}

}  // namespace
}  // namespace egs
