// tcgen05 / TMEM kernels for the three operators (sm_100a only).
//
// Common structure of both kernels (one CTA = one 128-row accumulator tile in tensor memory):
//   warps 0..7  producers: index-driven 16-byte cp.async row gathers from global memory into shared
//               memory, written directly in the 128-byte-swizzled layout the tensor core reads, through a
//               ring of `stages` buffers; afterwards the same warps run the epilogue (tcgen05.ld of the
//               accumulator, then vector stores or vector red.global.add.f32 into the destination rows)
//   warp 8      allocates tensor memory; one lane issues tcgen05.mma per stage and commits to mbarriers
// Stage hand-over uses mbarriers only: empty[s] (MMA completion -> producers), full[s] (data landed ->
// MMA lane), done (all MMAs -> epilogue).  Producers never wait for their own copies: after issuing a
// stage each thread executes cp.async.mbarrier.arrive.noinc, so the hardware arrives on full[s] when that
// thread's copies have landed and the producers run ahead by the whole ring.  (Strict float32 is the
// exception: it must pass the landed data through registers to split it, so there the producers wait for
// the copy group, split in place and arrive themselves.)  Every wait is bounded: when it runs out the
// thread sets the CTA's abort flag and EGS_STATUS_PIPELINE_TIMEOUT in the caller's status word, and all
// roles fall through to the common exit, where tensor memory is released.
//
// Shared-memory tile format (one format for every operand): rows of 128-byte segments.  Element
// (row r, 16-byte chunk c of the row) lives at
//     base + (c / 8) * seg_stride + (r / 8) * 1024 + (r % 8) * 128 + ((c % 8) ^ (r % 8)) * 16
// i.e. 8-row x 128-byte atoms with the hardware's 128B XOR swizzle, atoms of one segment column stacked
// 1024 bytes apart, segment columns seg_stride = rows*128 bytes apart.  Read with a K-major descriptor
// (rows = M or N index, SBO = 1024) the row is a contraction-contiguous operand; read with an MN-major
// descriptor (rows = contraction index, LBO = seg_stride, SBO = 1024) the same bytes are a transposed
// operand.  That is what lets gathered rows feed both  rows x W  (operators G, S) and  rows^T x rows
// (operator D) without a transposing copy, and never materialises the gathered [B,E,K,I] block.
// One exception: the tensor core reads MN-major 32-bit (TF32) operands only in the variant of this format
// whose XOR acts on 32-byte pairs with the row index modulo 4 (atoms of 4 rows; SBO = 512); float32 tiles
// that are consumed MN-major are written in that variant.
//
// float32 tensors: kind::tf32.  EGS_PREC_STRICT splits every operand chunk in shared memory into
// hi = top 19 bits and lo = tf32(x - hi) and issues lo*hi + hi*lo + hi*hi into the same accumulator, which
// restores ~fp32 product accuracy (the reference computes fp32 dots with allow_tf32=False,
// egs/triton_kernels.py:389).  16-bit tensors: kind::f16 with fp32 accumulation.
#include "egs_tcgen05.cuh"

namespace egs {

namespace {

// ------------------------------------------------------------------------------------------------
// Pipeline pieces shared by the two kernels
// ------------------------------------------------------------------------------------------------
struct Pipe {
  SmemHeader* hdr;
  volatile uint32_t* abort_flag;
  int32_t* status;
  uint32_t tiles0;        // shared-window address of stage 0
  uint32_t stage_bytes;
  int stages;
  int nk;                 // stages of work (contraction steps)
};

// One CTA-wide barrier: mbarrier init, abort check, tensor-memory allocation.  Returns the TMEM base.
__device__ __forceinline__ uint32_t pipe_setup(const Pipe& pp, uint32_t full_count, uint32_t tmem_cols, int tid, int warp) {
  SmemHeader* hdr = pp.hdr;
  if (tid == 0) {
    for (int s = 0; s < kMaxStages; ++s) {
      mbar_init(smem_u32(&hdr->full[s]), full_count);
      mbar_init(smem_u32(&hdr->empty[s]), 1);
    }
    mbar_init(smem_u32(&hdr->done), 1);
    mbar_init(smem_u32(&hdr->drain), 1);
    fence_mbar_init();
    // A launch that follows a timed-out one on the same status word does no work (keeps a broken pipeline
    // from costing one wait limit per wave of CTAs).
    hdr->abort_flag =
        (pp.status && (*reinterpret_cast<volatile int32_t*>(pp.status) & EGS_STATUS_PIPELINE_TIMEOUT)) ? 1u : 0u;
    if (smem_misaligned(hdr)) {
      hdr->abort_flag = 1u;
      if (pp.status) atomicOr(pp.status, EGS_STATUS_INTERNAL);
    }
  }
  if (warp == kProducerWarps) {
    tmem_alloc(smem_u32(&hdr->tmem_base), tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  return hdr->tmem_base;
}

__device__ __forceinline__ void pipe_teardown(const Pipe& pp, uint32_t tmem_base, uint32_t tmem_cols, int warp) {
  tc_fence_before();
  __syncthreads();
  if (warp == kProducerWarps) tmem_release(tmem_base, tmem_cols, smem_u32(&pp.hdr->drain), pp.abort_flag, threadIdx.x & 31);
}

// Common end of every producer variant: drain own copies, then wait (warp-uniformly) for the accumulator.
__device__ __forceinline__ bool producer_finish(const Pipe& pp, int lane, bool alive) {
  cp_async_wait_all();
  // all lanes of a warp must take the tcgen05.ld of the epilogue together: the decision is warp-uniform
  alive = __all_sync(0xffffffffu, alive);
  if (alive && pp.nk > 0) alive = mbar_wait_warp(smem_u32(&pp.hdr->done), 0u, pp.abort_flag, pp.status, lane);
  if (alive) tc_fence_after();
  return alive;
}

// Producer main loop.  issue(kt, stage_base) enqueues this thread's cp.async copies of stage kt;
// split(kt, stage_base) is the strict-mode in-place hi/lo pass over the same chunks.
template <bool STRICT, class Issue, class Split>
__device__ __forceinline__ bool run_producer(const Pipe& pp, int lane, Issue&& issue, Split&& split) {
  SmemHeader* hdr = pp.hdr;
  const int stages = pp.stages, nk = pp.nk;
  bool alive = true;
  if (!STRICT) {
    for (int kt = 0; kt < nk; ++kt) {
      const int slot = kt % stages, use = kt / stages;
      if (use > 0) alive = mbar_wait_warp(smem_u32(&hdr->empty[slot]), (use - 1) & 1, pp.abort_flag, pp.status, lane);
      if (!alive) break;
      issue(kt, pp.tiles0 + slot * pp.stage_bytes);
      cp_async_mbar_arrive_noinc(smem_u32(&hdr->full[slot]));
    }
  } else {
    const int dist = stages - 1;
    for (int kt = 0; kt < dist; ++kt) {
      if (kt < nk) issue(kt, pp.tiles0 + (kt % stages) * pp.stage_bytes);
      cp_async_commit();
    }
    for (int kc = 0; kc < nk; ++kc) {
      cp_async_wait_pending(dist - 1);
      if (alive) {
        split(kc, pp.tiles0 + (kc % stages) * pp.stage_bytes);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&hdr->full[kc % stages]));
      }
      const int kt = kc + dist;
      if (kt < nk && alive) {
        const int use = kt / stages;
        if (use > 0) alive = mbar_wait_warp(smem_u32(&hdr->empty[kt % stages]), (use - 1) & 1, pp.abort_flag, pp.status, lane);
        if (alive) issue(kt, pp.tiles0 + (kt % stages) * pp.stage_bytes);
      }
      cp_async_commit();
    }
  }
  return producer_finish(pp, lane, alive);
}

// hi/lo split of one 16-byte chunk of float32 values that already sits in the hi tile.  The tensor core reads a
// TF32 operand from the top 19 bits of each word and ignores the rest, so the raw float32 words ARE the hi
// operand; only lo = tf32(x - trunc19(x)) has to be written, to the lo tile.
__device__ __forceinline__ void split_store(uint32_t addr, uint32_t lo_offset, const uint4& x) {
  const uint32_t v[4] = {x.x, x.y, x.z, x.w};
  uint32_t lo[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float rem = __uint_as_float(v[i]) - __uint_as_float(v[i] & 0xFFFFE000u);
    lo[i] = (__float_as_uint(rem) + 0x1000u) & 0xFFFFE000u;   // round to tf32 (nearest, ties away) with integer ops
  }
  asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(addr + lo_offset), "r"(lo[0]), "r"(lo[1]), "r"(lo[2]), "r"(lo[3])
               : "memory");
}
__device__ __forceinline__ uint4 lds16(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
  return v;
}

// MMA lane main loop.  mma(ks, stage_base) issues the tcgen05.mma instructions of stage ks.
template <class Mma>
__device__ __forceinline__ void run_mma_lane(const Pipe& pp, Mma&& mma) {
  SmemHeader* hdr = pp.hdr;
  bool ok = true;
  for (int ks = 0; ks < pp.nk; ++ks) {
    const int slot = ks % pp.stages;
    ok = mbar_wait(smem_u32(&hdr->full[slot]), (ks / pp.stages) & 1, pp.abort_flag, pp.status);
    if (!ok) break;
    tc_fence_after();
    mma(ks, pp.tiles0 + slot * pp.stage_bytes);
    umma_commit(smem_u32(&hdr->empty[slot]));
  }
  if (ok && pp.nk > 0) umma_commit(smem_u32(&hdr->done));
}

// ------------------------------------------------------------------------------------------------
// Operators G and S.   grid = (row tiles, ceil(N/BN), E), or with expert_fastest (E, ceil(N/BN), row tiles).
//   Experts slowest: the CTAs in flight share one expert's weights and (for S) add to distinct token rows.
//   Experts fastest: the CTAs in flight work on the same few batch elements, so the token rows they gather
//   from or add to stay resident in L2 - chosen when those rows exceed L2 while all weights fit in it.
//   A rows (K-major): G gathers token rows through Ind, S reads slot rows
//   B = W[e]:  EGS_W_NC -> rows n, contraction contiguous (K-major);  EGS_W_CN -> rows c, n contiguous (MN-major)
//   epilogue:  G stores slot rows;  S adds to token rows with vector red.global.add.f32
// ------------------------------------------------------------------------------------------------
// MT = number of 128-row accumulator tiles per CTA (1 or 2).  With MT = 2 the CTA owns 256 expert rows: both
// accumulators are fed from the same W tile, which cuts the bytes loaded per flop by a third and lets a
// three-stage ring of one CTA per SM cover the load latency that two 2-stage CTAs cannot.
template <typename T, bool STRICT, bool SCATTER, int MT>
__global__ void __launch_bounds__(kThreads, MT == 2 ? 1 : 2) tensor_rowgemm_kernel(RowGemmParams p) {
  constexpr int kRows = kTileM * MT;        // expert rows per CTA
  constexpr int ES = sizeof(T);
  constexpr int KE = 128 / ES;        // contraction elements per stage (one 128-byte segment)
  constexpr int UK = 32 / ES;         // contraction elements per tcgen05.mma
  constexpr bool kMn32 = (ES == 4);   // MN-major 32-bit tiles use the 32-byte-granule swizzle
  constexpr uint32_t kMnLayout = kMn32 ? kSwizzle128Base32 : kSwizzle128;
  constexpr uint32_t kMnSbo = kMn32 ? 512u : 1024u;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  char* smem = reinterpret_cast<char*>(smem_raw);
  SmemHeader* hdr = reinterpret_cast<SmemHeader*>(smem);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int e = p.expert_fastest ? blockIdx.x : blockIdx.z;
  const int m0 = (p.expert_fastest ? blockIdx.z : blockIdx.x) * kRows;
  const int n0 = blockIdx.y * p.BN;
  const int bn = min(p.BN, ((p.N - n0) + 15) & ~15);       // MMA N of this tile (multiple of 16)
  const bool w_nc = (p.w_layout == EGS_W_NC);

  const uint32_t a_bytes = kRows * 128u;
  const int nseg_b = (p.BN * ES + 127) / 128;
  const uint32_t b_bytes = w_nc ? static_cast<uint32_t>(p.BN) * 128u : static_cast<uint32_t>(nseg_b) * KE * 128u;
  const uint32_t a_lo_off = a_bytes;                                   // strict: A_hi | A_lo | B_hi | B_lo
  const uint32_t b_off = STRICT ? 2u * a_bytes : a_bytes;
  const uint32_t b_lo_off = b_bytes;

  Pipe pp;
  pp.hdr = hdr;
  pp.abort_flag = &hdr->abort_flag;
  pp.status = p.status;
  pp.tiles0 = smem_u32(smem) + kHeaderBytes;
  pp.stage_bytes = (a_bytes + b_bytes) * (STRICT ? 2u : 1u);
  pp.stages = p.stages;
  pp.nk = (p.C + KE - 1) / KE;

  // ---- set-up ----
  if (tid < kRows) {
    const int m = m0 + tid;
    int ra = -1, ro = -1;
    if (m < p.M) {
      const int b = m / p.K, k = m - b * p.K;
      const int slot = (b * p.E + e) * p.K + k;
      const long long t = load_index(p.Ind, p.index_dtype, slot);
      if (t >= 0 && t < p.T) {
        const int tok = b * p.T + static_cast<int>(t);
        ra = SCATTER ? slot : tok;
        ro = SCATTER ? tok : slot;
      } else {
        if (p.status) atomicOr(p.status, EGS_STATUS_INDEX_OUT_OF_RANGE);
        if (!SCATTER) ro = slot;      // gather: the row is still written (zeros)
      }
    }
    hdr->row_a[tid] = ra;
    hdr->row_o[tid] = ro;
  }
  const uint32_t acc_cols = tmem_cols_for(p.BN);      // columns of one accumulator
  const uint32_t tmem_cols = acc_cols * MT;
  const uint32_t tmem_base = pipe_setup(pp, STRICT ? kProducerWarps : kProducerThreads, tmem_cols, tid, warp);
  const bool run = (hdr->abort_flag == 0u);

  if (!run) {
    // fall through to the common exit
  } else if (warp < kProducerWarps) {
    // =========================== producers ===========================
    const char* A = static_cast<const char*>(p.A);
    const char* W = static_cast<const char*>(p.W);
    const long long row_bytes_a = static_cast<long long>(p.C) * ES;

    // Every thread copies the same set of 16-byte chunks in every stage, only the contraction offset moves:
    // source pointers, destination offsets and validity are worked out once, the per-stage loop adds offsets.
    //   A: rows (tid/8) + 32*i, chunk tid%8            -> destination a_dst0 + i*4096
    //   B (EGS_W_NC): rows (tid/8) + 32*i, chunk tid%8 -> destination b_dst0 + i*4096
    //   B (EGS_W_CN): row r0 + i*rstep, chunk tid % cpr (when cpr divides 256; otherwise a generic walk)
    const int cc = tid & 7;
    const int r0 = tid >> 3;
    const uint32_t rc_dst0 = static_cast<uint32_t>(r0) * 128u + (static_cast<uint32_t>(cc ^ (r0 & 7)) << 4);
    const char* a_src[kRows / 32];
    uint32_t a_mask = 0;
#pragma unroll
    for (int i = 0; i < kRows / 32; ++i) {
      const int ra = hdr->row_a[r0 + 32 * i];
      a_src[i] = A + (ra >= 0 ? static_cast<long long>(ra) * row_bytes_a : 0ll) + cc * 16;
      if (ra >= 0) a_mask |= 1u << i;
    }
    // B, rows = n
    const int nb_iters = (p.BN + 31) / 32;
    const long long nc_stride = 32ll * row_bytes_a;
    const char* nc_src0 = W + (static_cast<long long>(e) * p.N + n0 + r0) * row_bytes_a + cc * 16;
    uint32_t nc_mask = 0;
    for (int i = 0; i < nb_iters; ++i)
      if (r0 + 32 * i < p.BN && n0 + r0 + 32 * i < p.N) nc_mask |= 1u << i;
    // B, rows = contraction index
    const int cpr = nseg_b * 8;
    const bool cn_fast = (kProducerThreads % cpr) == 0;
    const int cn_c = tid % cpr, cn_r0 = tid / cpr, cn_rstep = kProducerThreads / cpr;
    const long long row_bytes_w = static_cast<long long>(p.N) * ES;
    const bool cn_colvalid = static_cast<long long>(n0) * ES + cn_c * 16 < row_bytes_w;
    const char* cn_src0 = W + (static_cast<long long>(e) * p.C + cn_r0) * row_bytes_w + static_cast<long long>(n0) * ES + cn_c * 16;
    const long long cn_stride = static_cast<long long>(cn_rstep) * row_bytes_w;
    const uint32_t cn_dst_seg = static_cast<uint32_t>(cn_c >> 3) * (KE * 128u);

    // visits every 16-byte chunk this thread owns in stage `kt`:  f(dst_hi_addr, src, valid, is_b)
    auto for_each_chunk = [&](int kt, uint32_t stage_base, auto&& f) {
      const int k0 = kt * KE;
      const long long koff = static_cast<long long>(k0) * ES;
      const bool kvalid = koff + cc * 16 < row_bytes_a;
#pragma unroll
      for (int i = 0; i < kRows / 32; ++i)
        f(stage_base + rc_dst0 + i * 4096u, a_src[i] + koff, kvalid && ((a_mask >> i) & 1u), false);
      if (w_nc) {
        const char* src = nc_src0 + koff;
        for (int i = 0; i < nb_iters; ++i, src += nc_stride)
          if (r0 + 32 * i < p.BN) f(stage_base + b_off + rc_dst0 + i * 4096u, src, kvalid && ((nc_mask >> i) & 1u), true);
      } else if (cn_fast) {
        const char* src = cn_src0 + static_cast<long long>(k0) * row_bytes_w;
        for (int r = cn_r0; r < KE; r += cn_rstep, src += cn_stride) {
          const uint32_t dst = stage_base + b_off + cn_dst_seg + static_cast<uint32_t>(r) * 128u +
                               (kMn32 ? ((static_cast<uint32_t>(((cn_c & 7) >> 1) ^ (r & 3)) << 5) + (static_cast<uint32_t>(cn_c & 1) << 4))
                                      : (static_cast<uint32_t>((cn_c & 7) ^ (r & 7)) << 4));
          f(dst, src, cn_colvalid && (k0 + r) < p.C, true);
        }
      } else {
        const long long noff0 = static_cast<long long>(n0) * ES;
        for (int idx = tid; idx < KE * cpr; idx += kProducerThreads) {
          const int r = idx / cpr, c = idx - r * cpr;
          const long long noff = noff0 + c * 16;
          const char* src = W + (static_cast<long long>(e) * p.C + k0 + r) * row_bytes_w + noff;
          f(tile_addr<kMn32>(stage_base + b_off, KE * 128u, r, c), src, (k0 + r) < p.C && noff < row_bytes_w, true);
        }
      }
    };
    // Lean issue path for interior stages of full tiles (every row valid, the stage inside the contraction
    // range): no predicates, destination offsets are immediates, about two instructions per copy.
    const bool a_full = (a_mask == (1u << (kRows / 32)) - 1u);
    const bool nc_full = w_nc && (p.BN % 32 == 0) && (n0 + p.BN <= p.N);
    const bool cn_full = !w_nc && cn_fast && (KE % cn_rstep == 0) &&
                         (static_cast<long long>(n0) * ES + cpr * 16 <= row_bytes_w);
    const bool tile_full = a_full && (nc_full || cn_full);
    auto cn_swz = [&](int r) -> uint32_t {
      return kMn32 ? ((static_cast<uint32_t>(((cn_c & 7) >> 1) ^ (r & 3)) << 5) + (static_cast<uint32_t>(cn_c & 1) << 4))
                   : (static_cast<uint32_t>((cn_c & 7) ^ (r & 7)) << 4);
    };
    auto issue_full = [&](int kt, uint32_t stage_base) {
      const long long koff = static_cast<long long>(kt) * 128;
      const uint32_t da = stage_base + rc_dst0;
#pragma unroll
      for (int i = 0; i < kRows / 32; ++i) cp_async16_full(da + i * 4096u, a_src[i] + koff);
      if (w_nc) {
        const char* src = nc_src0 + koff;
        const uint32_t db = da + b_off;
        for (int i = 0; i < nb_iters; ++i, src += nc_stride) cp_async16_full(db + i * 4096u, src);
      } else {
        const char* src = cn_src0 + static_cast<long long>(kt * KE) * row_bytes_w;
        const uint32_t db = stage_base + b_off + cn_dst_seg;
        for (int r = cn_r0; r < KE; r += cn_rstep, src += cn_stride)
          cp_async16_full(db + static_cast<uint32_t>(r) * 128u + cn_swz(r), src);
      }
    };
    // strict float32: when this thread's chunk list has the fixed 4 + 4 shape the in-place hi/lo split reads all
    // of its chunks first (the loads pipeline) and only then splits and stores them
    const bool split_batched = STRICT && MT == 1 && (w_nc ? nb_iters <= 4 : (cn_fast && KE % cn_rstep == 0 && KE / cn_rstep <= 4));
    auto split_stage_batched = [&](int, uint32_t base) {
      uint32_t dst[8];
      bool on[8];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        dst[i] = base + rc_dst0 + i * 4096u;
        on[i] = true;
        if (w_nc) {
          dst[4 + i] = base + b_off + rc_dst0 + i * 4096u;
          on[4 + i] = i < nb_iters && r0 + 32 * i < p.BN;
        } else {
          const int rr = cn_r0 + i * cn_rstep;
          dst[4 + i] = base + b_off + cn_dst_seg + static_cast<uint32_t>(rr) * 128u +
                       (static_cast<uint32_t>(((cn_c & 7) >> 1) ^ (rr & 3)) << 5) + (static_cast<uint32_t>(cn_c & 1) << 4);
          on[4 + i] = rr < KE;
        }
      }
      uint4 r[8];
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (on[i]) r[i] = lds16(dst[i]);
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (on[i]) split_store(dst[i], i < 4 ? a_lo_off : b_lo_off, r[i]);
    };
    auto issue_stage = [&](int kt, uint32_t base) {
      if (tile_full && (kt + 1) * KE <= p.C) {
        issue_full(kt, base);
      } else {
        for_each_chunk(kt, base, [&](uint32_t dst, const char* src, bool v, bool) { cp_async16(dst, v ? src : W, v ? 16u : 0u); });
      }
    };
    bool alive;
    if (split_batched) alive = run_producer<STRICT>(pp, lane, issue_stage, split_stage_batched);
    else
    alive = run_producer<STRICT>(
        pp, lane,
        [&](int kt, uint32_t base) {
          if (tile_full && (kt + 1) * KE <= p.C) {
            issue_full(kt, base);
          } else {
            for_each_chunk(kt, base, [&](uint32_t dst, const char* src, bool v, bool) { cp_async16(dst, v ? src : W, v ? 16u : 0u); });
          }
        },
        [&](int kc, uint32_t base) {
          for_each_chunk(kc, base, [&](uint32_t dst, const char*, bool, bool is_b) {
            split_chunk(dst, is_b ? b_lo_off : a_lo_off);
          });
        });

    // =========================== epilogue ===========================
    // The stage ring is idle once `done` has completed: its first 32 KB serve as the warps' transpose tiles.
    if (alive) {
      const int lg = warp & 3, half = warp >> 2;
      const uint32_t tile = pp.tiles0 + static_cast<uint32_t>(warp) * 4096u;
      T* out = static_cast<T*>(p.Out);
      float* acc_rows = (ES == 2) ? p.acc : reinterpret_cast<float*>(p.Out);   // S: float32 rows being added to
      // 16-bit S: the planning flag says whether to add into the float32 rows or straight into the output
      const bool direct16 = SCATTER && ES == 2 && p.plan != nullptr && *p.plan == 0;
      const int nblk = (bn + 31) >> 5;
      // direct 16-bit adds go out in 64-column blocks (128-byte row segments) when the ring has room for the
      // eight 8 KB transpose tiles and the tile width is a multiple of 64
      const bool wide16 = direct16 && (bn % 64 == 0) && (pp.stages * pp.stage_bytes >= 8u * 8192u);
      // direct 16-bit adds as bulk reductions: every lane stages 128 bytes (64 columns) of its own row in the idle
      // ring and hands them to the copy engine (see the persistent variant)
      static_assert(2u * kBulkBufBytes <= 16384u, "two staging buffers per warp");
      const bool bulk16 = direct16 && p.bulk_epilogue && p.bias == nullptr && (pp.stages * pp.stage_bytes >= 8u * 2u * kBulkBufBytes);
      const T* bias_row = p.bias ? static_cast<const T*>(p.bias) + static_cast<long long>(e) * p.N : nullptr;
      if (bulk16) {
        if constexpr (ES == 2 && SCATTER) {
          const uint32_t my_stage = pp.tiles0 + static_cast<uint32_t>(warp) * (2u * kBulkBufBytes) + static_cast<uint32_t>(lane) * kBulkRowPitch;
          int q = 0;
          for (int mt = 0; mt < MT; ++mt) {
            const int ro = hdr->row_o[mt * kTileM + lg * 32 + lane];
            const uint32_t acc0 = tmem_base + (static_cast<uint32_t>(lg * 32) << 16) + mt * acc_cols;
            for (int c = half; c * 64 < bn; c += 2, ++q) {
              const uint32_t srow = my_stage + static_cast<uint32_t>(q & 1) * kBulkBufBytes;
              if (q >= 2) bulk_wait_read_1();
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                if (c * 64 + h * 32 < bn) {
                  uint32_t v[32];
                  tmem_ld32(acc0 + static_cast<uint32_t>(c * 64 + h * 32), v);
                  tmem_ld_wait();
#pragma unroll
                  for (int j = 0; j < 4; ++j)
                    asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(srow + h * 64u + j * 16u),
                                 "r"(pack2(out, v[8 * j], v[8 * j + 1])), "r"(pack2(out, v[8 * j + 2], v[8 * j + 3])),
                                 "r"(pack2(out, v[8 * j + 4], v[8 * j + 5])), "r"(pack2(out, v[8 * j + 6], v[8 * j + 7]))
                                 : "memory");
                }
              }
              fence_proxy_async_smem();
              const int col0 = n0 + c * 64;
              const int ncols = min(64, p.N - col0);
              if (ro >= 0 && ncols > 0)
                bulk_reduce_add(out + static_cast<long long>(ro) * p.N + col0, srow, static_cast<uint32_t>(ncols) * 2u);
              bulk_commit();
            }
          }
          bulk_wait_all();                               // shared memory must outlive the copy engine's reads
        }
      } else if (wide16) {
        const uint32_t tile8 = pp.tiles0 + static_cast<uint32_t>(warp) * 8192u;
        for (int mt = 0; mt < MT; ++mt) {
          for (int c = half; c < (bn >> 6); c += 2) {
            const int col0 = n0 + c * 64;
            warp_block_emit64(tmem_base + (static_cast<uint32_t>(lg * 32) << 16) + mt * acc_cols + static_cast<uint32_t>(c * 64), tile8,
                              lane, [&](int row, int cj, const uint32_t (&x)[8]) {
                                const int ro = hdr->row_o[mt * kTileM + lg * 32 + row];
                                const int col = col0 + cj;
                                if (ro >= 0 && col < p.N) {
                                  if (bias_row) {
                                    uint32_t y[8];
#pragma unroll
                                    for (int i = 0; i < 8; ++i) y[i] = x[i];
                                    add_bias4<T>(bias_row + col, y[0], y[1], y[2], y[3]);
                                    add_bias4<T>(bias_row + col + 4, y[4], y[5], y[6], y[7]);
                                    red8(out + static_cast<long long>(ro) * p.N + col, y);
                                  } else {
                                    red8(out + static_cast<long long>(ro) * p.N + col, x);
                                  }
                                }
                              });
          }
        }
      } else
      for (int mt = 0; mt < MT; ++mt) {
        for (int c = half; c < nblk; c += 2) {
          const int col0 = n0 + c * 32;
          warp_block_emit(tmem_base + (static_cast<uint32_t>(lg * 32) << 16) + mt * acc_cols + static_cast<uint32_t>(c * 32), tile,
                          lane, true, [&](int row, int cj, uint32_t x0, uint32_t x1, uint32_t x2, uint32_t x3) {
                            const int ro = hdr->row_o[mt * kTileM + lg * 32 + row];
                            const int col = col0 + cj;
                            if (ro >= 0 && col < p.N) {
                              const long long off = static_cast<long long>(ro) * p.N + col;
                              if (bias_row) add_bias4<T>(bias_row + col, x0, x1, x2, x3);
                              if (SCATTER) {
                                if (direct16) red4(out + off, x0, x1, x2, x3);
                                else red4(acc_rows + off, x0, x1, x2, x3);
                              } else {
                                store4(out + off, x0, x1, x2, x3);   // masked source rows were zero-filled: zeros
                              }
                            }
                          });
        }
      }
    }
  } else {
    // =========================== MMA issuer ===========================
    if (lane == 0) {
      const uint32_t idesc = make_idesc(Elem<T>::fmt, 0u, w_nc ? 0u : 1u, kTileM, static_cast<uint32_t>(bn));
      const uint32_t b_lbo = w_nc ? 16u : KE * 128u;
      const uint32_t b_sbo = w_nc ? 1024u : kMnSbo;
      const uint32_t b_lay = w_nc ? kSwizzle128 : kMnLayout;
      const uint32_t b_step = w_nc ? 32u : UK * 128u;
      // descriptors differ between MMAs only in the start-address field (low 14 bits of the low word, in
      // 16-byte units): build them once per stage and advance with an add
      const uint64_t a_adv = 32u >> 4, b_adv = b_step >> 4;
      run_mma_lane(pp, [&](int ks, uint32_t a_hi) {
        const uint32_t b_hi = a_hi + b_off;
        const int kq0 = 0, kq1 = min(KE / UK, (p.C - ks * KE + UK - 1) / UK);
        uint64_t ad[MT], adl[MT];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          ad[mt] = make_smem_desc(a_hi + mt * (kTileM * 128u), 16u, 1024u) + kq0 * a_adv;
          adl[mt] = STRICT ? make_smem_desc(a_hi + mt * (kTileM * 128u) + a_lo_off, 16u, 1024u) + kq0 * a_adv : 0ull;
        }
        uint64_t bd = make_smem_desc(b_hi, b_lbo, b_sbo, b_lay) + kq0 * b_adv;
        uint64_t bdl = STRICT ? make_smem_desc(b_hi + b_lo_off, b_lbo, b_sbo, b_lay) + kq0 * b_adv : 0ull;
        for (int kq = kq0; kq < kq1; ++kq) {
          const uint32_t acc = (ks > 0 || kq > 0) ? 1u : 0u;
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            const uint32_t d = tmem_base + mt * acc_cols;
            if (STRICT) {
              umma<Elem<T>::tf32>(d, adl[mt], bd, idesc, acc);
              umma<Elem<T>::tf32>(d, ad[mt], bdl, idesc, 1u);
              umma<Elem<T>::tf32>(d, ad[mt], bd, idesc, 1u);
            } else {
              umma<Elem<T>::tf32>(d, ad[mt], bd, idesc, acc);
            }
            ad[mt] += a_adv;
            adl[mt] += a_adv;
          }
          bd += b_adv;
          bdl += b_adv;
        }
      });
    }
    __syncwarp();
  }
  pipe_teardown(pp, tmem_base, tmem_cols, warp);
}

// ------------------------------------------------------------------------------------------------
// Operators G and S, persistent variant.   grid = min(#SMs, row blocks) CTAs of 17 warps.
//   A row block is one (expert, 128 expert rows) pair; a CTA walks row blocks blockIdx.x, +gridDim.x, ... and, inside
//   a row block, all N tiles.  The stage ring never drains between tiles, the accumulator is double-buffered in
//   tensor memory, and dedicated epilogue warps drain tile t while the tensor core works on tile t+1:
//     warps 0..7   producers (cp.async row gathers, hardware arrive on full[s])
//     warps 8..15  epilogue  (tcgen05.ld -> shared-memory transpose -> stores / red.global.add)
//     warp  16     TMEM allocation; one lane issues tcgen05.mma and commits to empty[s] and acc_full[b]
//   Short contractions with wide outputs (the scatter operator) are where this matters: with one CTA per tile
//   their time goes into the per-tile latency chain (set-up, first loads, a 2-stage ring, an epilogue nothing
//   overlaps), not into tensor work or atomics.
//   No shared row tables: every producer thread looks up the token rows of the four tile rows it copies, every
//   epilogue warp those of its 32 lanes, so the roles never have to meet at a CTA-wide barrier after set-up.
//   Non-strict arithmetic only (bf16 / fp16 / single TF32 product).
// ------------------------------------------------------------------------------------------------
constexpr int kPersistMaxEpilogueWarps = 8;
constexpr uint32_t kPersistHeaderBytes = 1024;
// Warp split: 8 producer + 8 epilogue warps.  (Measured: 4 producer warps starve the ring; 16 epilogue warps do not
// help because the transpose tiles then cost a ring stage and shared-memory bandwidth is what they compete for.)
template <bool SCATTER> struct PersistShape {
  static constexpr int kProducerWarps = 8;
  static constexpr int kEpilogueWarps = 8;
  static constexpr int kThreads = (kProducerWarps + kEpilogueWarps + 1) * 32;
};

struct __align__(16) PersistHeader {
  unsigned long long full[kMaxStages];
  unsigned long long empty[kMaxStages];
  unsigned long long acc_full[2];
  unsigned long long acc_empty[2];
  unsigned long long drain;
  uint32_t tmem_base;
  uint32_t abort_flag;
};
static_assert(sizeof(PersistHeader) <= kPersistHeaderBytes, "header does not fit");

struct RowBlock {
  int e, m0;
};
__device__ __forceinline__ RowBlock row_block_of(const RowGemmParams& p, int rb, int m_tiles) {
  RowBlock r;
  if (p.expert_fastest) {
    r.e = rb % p.E;
    r.m0 = (rb / p.E) * kTileM;
  } else {
    r.m0 = (rb % m_tiles) * kTileM;
    r.e = rb / m_tiles;
  }
  return r;
}
// Source / destination row of expert row m of expert e (-1 = masked).  G: source token row, destination slot row;
// S: source slot row, destination token row.
template <bool SCATTER>
__device__ __forceinline__ void lookup_rows(const RowGemmParams& p, int e, int m, int& src_row, int& dst_row, bool report) {
  src_row = -1;
  dst_row = -1;
  if (m >= p.M) return;
  const int b = m / p.K, k = m - b * p.K;
  const int slot = (b * p.E + e) * p.K + k;
  const long long t = load_index(p.Ind, p.index_dtype, slot);
  if (t >= 0 && t < p.T) {
    const int tok = b * p.T + static_cast<int>(t);
    src_row = SCATTER ? slot : tok;
    dst_row = SCATTER ? tok : slot;
  } else {
    if (report && p.status) atomicOr(p.status, EGS_STATUS_INDEX_OUT_OF_RANGE);
    if (!SCATTER) dst_row = slot;      // gather: the row is still written (zeros)
  }
}

template <typename T, bool SCATTER>
__global__ void __launch_bounds__(PersistShape<SCATTER>::kThreads, 1) tensor_rowgemm_persistent_kernel(RowGemmParams p) {
  constexpr int kPersistProducerWarps = PersistShape<SCATTER>::kProducerWarps;
  constexpr int kPersistEpilogueWarps = PersistShape<SCATTER>::kEpilogueWarps;
  constexpr int PT = kPersistProducerWarps * 32;     // producer threads
  constexpr int RS = PT / 8;                         // tile rows covered by one pass of the producers (8 threads per row)
  constexpr int ES = sizeof(T);
  constexpr int KE = 128 / ES;        // contraction elements per stage (one 128-byte segment)
  constexpr int UK = 32 / ES;         // contraction elements per tcgen05.mma
  constexpr bool kMn32 = (ES == 4);
  constexpr uint32_t kMnLayout = kMn32 ? kSwizzle128Base32 : kSwizzle128;
  constexpr uint32_t kMnSbo = kMn32 ? 512u : 1024u;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  PersistHeader* hdr = reinterpret_cast<PersistHeader*>(smem_raw);
  const uint32_t smem0 = smem_u32(smem_raw);
  const uint32_t xpose0 = smem0 + kPersistHeaderBytes;                             // 8 transpose tiles of 4 KB
  // per epilogue warp: a 4 KB transpose tile, or the two staging buffers of the bulk adds (the tile fits in them)
  const uint32_t xpose_tile = p.bulk_epilogue ? 2u * kBulkBufBytes : 4096u;
  const uint32_t tiles0 = xpose0 + ((kPersistMaxEpilogueWarps * xpose_tile + 1023u) & ~1023u);   // stage ring

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool w_nc = (p.w_layout == EGS_W_NC);
  const int m_tiles = (p.M + kTileM - 1) / kTileM;
  const int n_tiles = (p.N + p.BN - 1) / p.BN;
  const int row_blocks = p.E * m_tiles;
  const int stages = p.stages;
  const int nk = (p.C + KE - 1) / KE;
  const uint32_t a_bytes = kTileM * 128u;
  const int nseg_b = (p.BN * ES + 127) / 128;
  const uint32_t b_bytes = w_nc ? static_cast<uint32_t>(p.BN) * 128u : static_cast<uint32_t>(nseg_b) * KE * 128u;
  const uint32_t stage_bytes = a_bytes + b_bytes;
  const uint32_t b_off = a_bytes;
  const uint32_t acc_cols = tmem_cols_for(p.BN);
  const uint32_t tmem_cols = 2u * acc_cols;
  volatile uint32_t* abort_flag = &hdr->abort_flag;

  // ---- set-up: barriers, abort check, tensor memory (the only CTA-wide barrier before the exit) ----
  if (tid == 0) {
    for (int s = 0; s < kMaxStages; ++s) {
      mbar_init(smem_u32(&hdr->full[s]), kPersistProducerWarps * 32);
      mbar_init(smem_u32(&hdr->empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&hdr->acc_full[b]), 1);
      mbar_init(smem_u32(&hdr->acc_empty[b]), kPersistEpilogueWarps);
    }
    mbar_init(smem_u32(&hdr->drain), 1);
    fence_mbar_init();
    hdr->abort_flag = (p.status && (*reinterpret_cast<volatile int32_t*>(p.status) & EGS_STATUS_PIPELINE_TIMEOUT)) ? 1u : 0u;
    if (smem_misaligned(smem_raw)) {
      hdr->abort_flag = 1u;
      if (p.status) atomicOr(p.status, EGS_STATUS_INTERNAL);
    }
  }
  const int mma_warp = kPersistProducerWarps + kPersistEpilogueWarps;
  if (warp == mma_warp) {
    tmem_alloc(smem_u32(&hdr->tmem_base), tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = hdr->tmem_base;
  const bool run = (hdr->abort_flag == 0u);

  if (!run) {
    // fall through to the common exit
  } else if (warp < kPersistProducerWarps) {
    // =========================== producers ===========================
    const char* A = static_cast<const char*>(p.A);
    const char* W = static_cast<const char*>(p.W);
    const long long row_bytes_a = static_cast<long long>(p.C) * ES;
    const long long row_bytes_w = static_cast<long long>(p.N) * ES;
    const int cc = tid & 7, r0 = tid >> 3;
    const uint32_t rc_dst0 = static_cast<uint32_t>(r0) * 128u + (static_cast<uint32_t>(cc ^ (r0 & 7)) << 4);
    const int nb_iters = (p.BN + RS - 1) / RS;
    const long long nc_stride = static_cast<long long>(RS) * row_bytes_a;
    const int cpr = nseg_b * 8;
    const bool cn_fast = (PT % cpr) == 0;
    const int cn_c = tid % cpr, cn_r0 = tid / cpr, cn_rstep = PT / cpr;
    const long long cn_stride = static_cast<long long>(cn_rstep) * row_bytes_w;
    const uint32_t cn_dst_seg = static_cast<uint32_t>(cn_c >> 3) * (KE * 128u);
    auto mn_swz = [](int c, int r) -> uint32_t {
      return kMn32 ? ((static_cast<uint32_t>(((c & 7) >> 1) ^ (r & 3)) << 5) + (static_cast<uint32_t>(c & 1) << 4))
                   : (static_cast<uint32_t>((c & 7) ^ (r & 7)) << 4);
    };
    const uint32_t cn_dst0 = cn_dst_seg + static_cast<uint32_t>(cn_r0) * 128u + mn_swz(cn_c, cn_r0);
    const bool cn_shape_ok = cn_fast && (KE % cn_rstep == 0) && (cn_rstep % 8 == 0 || kMn32);
    bool alive = true;
    int g = 0;                                   // stages issued so far by this CTA (ring position)
    for (int rb = blockIdx.x; rb < row_blocks && alive; rb += gridDim.x) {
      const RowBlock blk = row_block_of(p, rb, m_tiles);
      const char* a_src[kTileM / RS];
      uint32_t a_mask = 0;
      int src_rows[kTileM / RS];
      if (SCATTER) {
        // the source rows of S are the slot rows themselves: no index is read here (a slot whose index is out of range
        // is dropped by the epilogue, which has no destination row for it)
#pragma unroll
        for (int i = 0; i < kTileM / RS; ++i) {
          const int m = blk.m0 + r0 + RS * i;
          const int b = m / p.K, k = m - b * p.K;
          src_rows[i] = (m < p.M) ? (b * p.E + blk.e) * p.K + k : -1;
        }
      } else {
        // all index loads are issued before the first one is looked at
        long long tk[kTileM / RS];
        int brow[kTileM / RS];
#pragma unroll
        for (int i = 0; i < kTileM / RS; ++i) {
          const int m = blk.m0 + r0 + RS * i;
          const bool on = m < p.M;
          const int b = on ? m / p.K : 0, k = on ? m - b * p.K : 0;
          brow[i] = on ? b * p.T : -1;
          tk[i] = load_index(p.Ind, p.index_dtype, static_cast<long long>(b * p.E + blk.e) * p.K + k);
        }
#pragma unroll
        for (int i = 0; i < kTileM / RS; ++i)
          src_rows[i] = (brow[i] >= 0 && tk[i] >= 0 && tk[i] < p.T) ? brow[i] + static_cast<int>(tk[i]) : -1;
      }
#pragma unroll
      for (int i = 0; i < kTileM / RS; ++i) {
        a_src[i] = A + (src_rows[i] >= 0 ? static_cast<long long>(src_rows[i]) * row_bytes_a : 0ll) + cc * 16;
        if (src_rows[i] >= 0) a_mask |= 1u << i;
      }
      const bool a_full = (a_mask == (1u << (kTileM / RS)) - 1u);
      for (int nt = 0; nt < n_tiles && alive; ++nt) {
        const int n0 = nt * p.BN;
        const char* nc_src0 = W + (static_cast<long long>(blk.e) * p.N + n0 + r0) * row_bytes_a + cc * 16;
        uint32_t nc_mask = 0;
        for (int i = 0; i < nb_iters; ++i)
          if (r0 + RS * i < p.BN && n0 + r0 + RS * i < p.N) nc_mask |= 1u << i;
        const char* cn_src0 =
            W + (static_cast<long long>(blk.e) * p.C + cn_r0) * row_bytes_w + static_cast<long long>(n0) * ES + cn_c * 16;
        const bool nc_full = w_nc && (p.BN % RS == 0) && (n0 + p.BN <= p.N);
        const bool cn_full = !w_nc && cn_shape_ok && (static_cast<long long>(n0) * ES + cpr * 16 <= row_bytes_w);
        const bool tile_full = a_full && (nc_full || cn_full);
        for (int kt = 0; kt < nk; ++kt, ++g) {
          const int slot = g % stages, use = g / stages;
          if (use > 0) alive = mbar_wait_warp(smem_u32(&hdr->empty[slot]), (use - 1) & 1, abort_flag, p.status, lane);
          if (!alive) break;
          const uint32_t base = tiles0 + slot * stage_bytes;
          const int k0 = kt * KE;
          const long long koff = static_cast<long long>(k0) * ES;
          if (tile_full && k0 + KE <= p.C) {
            // interior stage of a full tile: no predicates, immediate destination offsets
            const uint32_t da = base + rc_dst0;
#pragma unroll
            for (int i = 0; i < kTileM / RS; ++i) cp_async16_full(da + i * (RS * 128u), a_src[i] + koff);
            if (w_nc) {
              const char* src = nc_src0 + koff;
              const uint32_t db = da + b_off;
              for (int i = 0; i < nb_iters; ++i, src += nc_stride) cp_async16_full(db + i * (RS * 128u), src);
            } else {
              const char* src = cn_src0 + static_cast<long long>(k0) * row_bytes_w;
              const uint32_t db = base + b_off + cn_dst0;
              const uint32_t dstep = static_cast<uint32_t>(cn_rstep) * 128u;
              for (int r = cn_r0, i = 0; r < KE; r += cn_rstep, ++i, src += cn_stride) cp_async16_full(db + i * dstep, src);
            }
          } else {
            const bool kvalid = koff + cc * 16 < row_bytes_a;
#pragma unroll
            for (int i = 0; i < kTileM / RS; ++i) {
              const bool v = kvalid && ((a_mask >> i) & 1u);
              cp_async16(base + rc_dst0 + i * (RS * 128u), v ? a_src[i] + koff : A, v ? 16u : 0u);
            }
            if (w_nc) {
              const char* src = nc_src0 + koff;
              for (int i = 0; i < nb_iters; ++i, src += nc_stride) {
                if (r0 + RS * i >= p.BN) break;
                const bool v = kvalid && ((nc_mask >> i) & 1u);
                cp_async16(base + b_off + rc_dst0 + i * (RS * 128u), v ? src : W, v ? 16u : 0u);
              }
            } else {
              const long long noff0 = static_cast<long long>(n0) * ES;
              for (int idx = tid; idx < KE * cpr; idx += PT) {
                const int r = idx / cpr, c = idx - r * cpr;
                const long long noff = noff0 + c * 16;
                const bool v = (k0 + r) < p.C && noff < row_bytes_w;
                const char* src = W + (static_cast<long long>(blk.e) * p.C + k0 + r) * row_bytes_w + noff;
                cp_async16(tile_addr<kMn32>(base + b_off, KE * 128u, r, c), v ? src : W, v ? 16u : 0u);
              }
            }
          }
          cp_async_mbar_arrive_noinc(smem_u32(&hdr->full[slot]));
        }
      }
    }
    cp_async_wait_all();
  } else if (warp < kPersistProducerWarps + kPersistEpilogueWarps) {
    // =========================== epilogue ===========================
    const int ew = warp - kPersistProducerWarps;
    constexpr int kColGroups = kPersistEpilogueWarps / 4;
    const int lg = ew & 3, half = ew >> 2;               // TMEM lane group of this warp, which share of the column blocks
    const uint32_t tile = xpose0 + static_cast<uint32_t>(ew) * xpose_tile;
    T* out = static_cast<T*>(p.Out);
    float* acc_rows = (ES == 2) ? p.acc : reinterpret_cast<float*>(p.Out);   // S: float32 rows being added to
    const bool direct16 = SCATTER && ES == 2 && p.plan != nullptr && *p.plan == 0;
    // bulk adds (direct 16-bit scatter): every lane stages 128 bytes of its own row and hands them to the copy
    // engine - no transpose, no shuffles, and the warp does not wait on the load/store unit.  (For float32 rows
    // the same scheme needs twice the operations per column and measured slower than the transposed reds.)
    const bool bulk = direct16 && p.bulk_epilogue && p.bias == nullptr;
    const uint32_t my_stage = tile + static_cast<uint32_t>(lane) * kBulkRowPitch;
    int q = 0;                                           // bulk groups committed so far by this thread
    bool alive = true;
    int t = 0;                                           // tiles finished so far by this CTA
    for (int rb = blockIdx.x; rb < row_blocks && alive; rb += gridDim.x) {
      const RowBlock blk = row_block_of(p, rb, m_tiles);
      int src_row, my_ro;                                // destination row of tile row lg*32 + lane
      lookup_rows<SCATTER>(p, blk.e, blk.m0 + lg * 32 + lane, src_row, my_ro, half == 0);
      for (int nt = 0; nt < n_tiles && alive; ++nt, ++t) {
        const int n0 = nt * p.BN;
        const int bn = min(p.BN, ((p.N - n0) + 15) & ~15);
        const int buf = t & 1;
        alive = mbar_wait_warp(smem_u32(&hdr->acc_full[buf]), (t >> 1) & 1, abort_flag, p.status, lane);
        if (!alive) break;
        tc_fence_after();
        const int nblk = (bn + 31) >> 5;
        if (bulk) {
          const uint32_t acc0 = tmem_base + (static_cast<uint32_t>(lg * 32) << 16) + buf * acc_cols;
          if constexpr (ES == 2) {
            // 64 columns = 128 bytes of a 16-bit row per block
            for (int c = half; c * 64 < bn; c += kColGroups, ++q) {
              const uint32_t srow = my_stage + static_cast<uint32_t>(q & 1) * kBulkBufBytes;
              if (q >= 2) bulk_wait_read_1();            // the group that used this buffer two blocks ago has been read
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                if (c * 64 + h * 32 < bn) {
                  uint32_t v[32];
                  tmem_ld32(acc0 + static_cast<uint32_t>(c * 64 + h * 32), v);
                  tmem_ld_wait();
#pragma unroll
                  for (int j = 0; j < 4; ++j)
                    asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(srow + h * 64u + j * 16u),
                                 "r"(pack2(out, v[8 * j], v[8 * j + 1])), "r"(pack2(out, v[8 * j + 2], v[8 * j + 3])),
                                 "r"(pack2(out, v[8 * j + 4], v[8 * j + 5])), "r"(pack2(out, v[8 * j + 6], v[8 * j + 7]))
                                 : "memory");
                }
              }
              fence_proxy_async_smem();
              const int col0 = n0 + c * 64;
              const int ncols = min(64, p.N - col0);
              if (my_ro >= 0 && ncols > 0)
                bulk_reduce_add(out + static_cast<long long>(my_ro) * p.N + col0, srow, static_cast<uint32_t>(ncols) * 2u);
              bulk_commit();
            }
          }
        } else
        for (int c = half; c < nblk; c += kColGroups) {
          const int col0 = n0 + c * 32;
          warp_block_emit(tmem_base + (static_cast<uint32_t>(lg * 32) << 16) + buf * acc_cols + static_cast<uint32_t>(c * 32), tile, lane,
                          true, [&](int row, int cj, uint32_t x0, uint32_t x1, uint32_t x2, uint32_t x3) {
                            const int ro = __shfl_sync(0xffffffffu, my_ro, row);
                            const int col = col0 + cj;
                            if (ro >= 0 && col < p.N) {
                              const long long off = static_cast<long long>(ro) * p.N + col;
                              if (p.bias) add_bias4<T>(static_cast<const T*>(p.bias) + static_cast<long long>(blk.e) * p.N + col, x0, x1, x2, x3);
                              if (SCATTER) {
                                if (direct16) red4(out + off, x0, x1, x2, x3);
                                else red4(acc_rows + off, x0, x1, x2, x3);
                              } else {
                                store4(out + off, x0, x1, x2, x3);
                              }
                            }
                          });
        }
        // hand the accumulator buffer back to the MMA lane
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&hdr->acc_empty[buf]));
      }
    }
    if (bulk) bulk_wait_all();                           // shared memory must outlive the copy engine's reads
  } else {
    // =========================== MMA issuer ===========================
    if (lane == 0) {
      const uint32_t b_lbo = w_nc ? 16u : KE * 128u;
      const uint32_t b_sbo = w_nc ? 1024u : kMnSbo;
      const uint32_t b_lay = w_nc ? kSwizzle128 : kMnLayout;
      const uint64_t a_adv = 32u >> 4, b_adv = (w_nc ? 32u : UK * 128u) >> 4;
      bool ok = true;
      int g = 0, t = 0;
      for (int rb = blockIdx.x; rb < row_blocks && ok; rb += gridDim.x) {
        for (int nt = 0; nt < n_tiles && ok; ++nt, ++t) {
          const int n0 = nt * p.BN;
          const int bn = min(p.BN, ((p.N - n0) + 15) & ~15);
          const uint32_t idesc = make_idesc(Elem<T>::fmt, 0u, w_nc ? 0u : 1u, kTileM, static_cast<uint32_t>(bn));
          const int buf = t & 1;
          if (t >= 2) {
            ok = mbar_wait(smem_u32(&hdr->acc_empty[buf]), ((t >> 1) - 1) & 1, abort_flag, p.status);
            if (!ok) break;
            tc_fence_after();
          }
          const uint32_t d = tmem_base + buf * acc_cols;
          for (int ks = 0; ks < nk; ++ks, ++g) {
            const int slot = g % stages;
            ok = mbar_wait(smem_u32(&hdr->full[slot]), (g / stages) & 1, abort_flag, p.status);
            if (!ok) break;
            tc_fence_after();
            const uint32_t a_hi = tiles0 + slot * stage_bytes;
            uint64_t ad = make_smem_desc(a_hi, 16u, 1024u);
            uint64_t bd = make_smem_desc(a_hi + b_off, b_lbo, b_sbo, b_lay);
            const int krem = p.C - ks * KE;
            const int nkq = min(KE / UK, (krem + UK - 1) / UK);
            for (int kq = 0; kq < nkq; ++kq) {
              umma<Elem<T>::tf32>(d, ad, bd, idesc, (ks > 0 || kq > 0) ? 1u : 0u);
              ad += a_adv;
              bd += b_adv;
            }
            umma_commit(smem_u32(&hdr->empty[slot]));
          }
          if (ok) umma_commit(smem_u32(&hdr->acc_full[buf]));
        }
      }
    }
    __syncwarp();
  }

  // ---- common exit ----
  tc_fence_before();
  __syncthreads();
  if (warp == mma_warp) tmem_release(tmem_base, tmem_cols, smem_u32(&hdr->drain), abort_flag, lane);
}

// ------------------------------------------------------------------------------------------------
// Operator D.   grid = (ceil(FG/128), ceil(FD/BN), E*splits)
//   accumulator tile P[f, g]: TMEM lane = f (feature of the gathered rows), column = g
//   A = gathered token rows of Xsrc, B = slot rows of Ysrc; both consumed MN-major (rows = contraction)
//   The token row of every contraction row this CTA owns is looked up once into a shared-memory table.
//   splits == 1: the tile is stored in the output dtype; splits > 1: red.global.add.f32 into p.acc
//   MT = 128-feature accumulator tiles per CTA over FG (1 or 2).  With MT = 2 both accumulators are fed from
//   the same B tile: a third fewer bytes loaded per flop, which is what bounds this kernel once the contraction
//   is long (the loads of two 128 x 256 CTAs per SM top out well below the tensor rate).
// ------------------------------------------------------------------------------------------------
template <typename T, bool STRICT, int MT>
__global__ void __launch_bounds__(kThreads, MT == 2 ? 1 : 2) tensor_dweight_kernel(DWeightParams p) {
  constexpr int ES = sizeof(T);
  constexpr int KR = 128 / ES;          // contraction rows per stage (4 MMAs of UK rows)
  constexpr int UK = 32 / ES;           // contraction rows per tcgen05.mma
  constexpr int NSEG_A = ES * MT;       // 128*MT features * ES bytes / 128
  constexpr int CPR_A = NSEG_A * 8;     // 16-byte chunks per A row
  constexpr bool kMn32 = (ES == 4);     // MN-major 32-bit tiles use the 32-byte-granule swizzle
  constexpr uint32_t kMnLayout = kMn32 ? kSwizzle128Base32 : kSwizzle128;
  constexpr uint32_t kMnSbo = kMn32 ? 512u : 1024u;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  char* smem = reinterpret_cast<char*>(smem_raw);
  SmemHeader* hdr = reinterpret_cast<SmemHeader*>(smem);
  int* row_tok = reinterpret_cast<int*>(smem + kHeaderBytesD);    // [rows_per_split] token row or -1
  const uint32_t table_bytes = (static_cast<uint32_t>(p.rows_per_split) * 4u + 1023u) & ~1023u;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int e = blockIdx.z / p.splits;
  const int split = blockIdx.z - e * p.splits;
  const int f0 = blockIdx.x * (kTileM * MT);
  const int g0 = blockIdx.y * p.BN;
  const int bn = min(p.BN, ((p.FD - g0) + 15) & ~15);
  const int m_begin = split * p.rows_per_split;
  const int m_end = min(p.M, m_begin + p.rows_per_split);
  const int rows = max(0, m_end - m_begin);

  const int nseg_b = (p.BN * ES + 127) / 128;
  const uint32_t seg_stride = KR * 128u;
  const uint32_t a_bytes = NSEG_A * seg_stride;
  const uint32_t b_bytes = static_cast<uint32_t>(nseg_b) * seg_stride;
  const uint32_t a_lo_off = a_bytes;
  const uint32_t b_off = STRICT ? 2u * a_bytes : a_bytes;
  const uint32_t b_lo_off = b_bytes;

  Pipe pp;
  pp.hdr = hdr;
  pp.abort_flag = &hdr->abort_flag;
  pp.status = p.status;
  pp.tiles0 = smem_u32(smem) + kHeaderBytesD + table_bytes;
  pp.stage_bytes = (a_bytes + b_bytes) * (STRICT ? 2u : 1u);
  pp.stages = p.stages;
  pp.nk = (rows + KR - 1) / KR;

  // ---- set-up: token-row table (coalesced reads of Ind), barriers, tensor memory ----
  // (eight index loads are in flight per thread before the first is looked at: one load per round trip would make
  // this table the longest part of the set-up)
  for (int i0 = tid; i0 < rows; i0 += 8 * kThreads) {
    long long tk[8];
    int brow[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int i = i0 + j * kThreads;
      const bool on = i < rows;
      const int m = m_begin + (on ? i : 0);
      const int b = m / p.K, k = m - b * p.K;
      brow[j] = on ? b * p.T : -1;
      tk[j] = load_index(p.Ind, p.index_dtype, static_cast<long long>(b * p.E + e) * p.K + k);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (brow[j] >= 0) {
        int tok = -1;
        if (tk[j] >= 0 && tk[j] < p.T) tok = brow[j] + static_cast<int>(tk[j]);
        else if (p.status) atomicOr(p.status, EGS_STATUS_INDEX_OUT_OF_RANGE);
        row_tok[i0 + j * kThreads] = tok;
      }
    }
  }
  const uint32_t acc_cols = tmem_cols_for(p.BN);
  const uint32_t tmem_cols = acc_cols * MT;
  const uint32_t tmem_base = pipe_setup(pp, STRICT ? kProducerWarps : kProducerThreads, tmem_cols, tid, warp);
  const bool run = (hdr->abort_flag == 0u);

  if (!run) {
    // fall through to the common exit
  } else if (warp < kProducerWarps) {
    const char* Xs = static_cast<const char*>(p.Xsrc);
    const char* Ys = static_cast<const char*>(p.Ysrc);
    const long long row_bytes_g = static_cast<long long>(p.FG) * ES;
    const long long row_bytes_d = static_cast<long long>(p.FD) * ES;
    const int cpr_b = nseg_b * 8;
    // Per-thread chunk walk, fixed for every stage (see the row kernel): A rows a_r0 + i*a_rstep with chunk
    // tid % CPR_A; B rows b_r0 + i*b_rstep with chunk tid % cpr_b when cpr_b divides 256.
    constexpr int a_rstep = kProducerThreads / CPR_A;
    const int a_c = tid % CPR_A, a_r0 = tid / CPR_A;
    const bool a_colvalid = static_cast<long long>(f0) * ES + a_c * 16 < row_bytes_g;
    const char* a_col = Xs + static_cast<long long>(f0) * ES + a_c * 16;
    const uint32_t a_dst_seg = static_cast<uint32_t>(a_c >> 3) * seg_stride;
    const bool b_fast = (kProducerThreads % cpr_b) == 0;
    const int b_c = tid % cpr_b, b_r0 = tid / cpr_b, b_rstep = kProducerThreads / cpr_b;
    const bool b_colvalid = static_cast<long long>(g0) * ES + b_c * 16 < row_bytes_d;
    const char* b_col = Ys + static_cast<long long>(g0) * ES + b_c * 16;
    const uint32_t b_dst_seg = static_cast<uint32_t>(b_c >> 3) * seg_stride;
    auto swz = [](int c, int r) -> uint32_t {
      return kMn32 ? ((static_cast<uint32_t>(((c & 7) >> 1) ^ (r & 3)) << 5) + (static_cast<uint32_t>(c & 1) << 4))
                   : (static_cast<uint32_t>((c & 7) ^ (r & 7)) << 4);
    };

    auto for_each_chunk = [&](int kt, uint32_t stage_base, bool want_src, auto&& f) {
      const int i0 = kt * KR;
      // A: KR contraction rows x CPR_A chunks of the 128 gathered features
#pragma unroll
      for (int r = a_r0; r < KR; r += a_rstep) {
        const int tok = (want_src && i0 + r < rows) ? row_tok[i0 + r] : -1;
        const bool v = a_colvalid && tok >= 0;
        f(stage_base + a_dst_seg + static_cast<uint32_t>(r) * 128u + swz(a_c, r),
          a_col + (v ? static_cast<long long>(tok) * row_bytes_g : 0ll), v, false);
      }
      // B: KR contraction rows x cpr_b chunks of the BN direct features
      if (b_fast) {
        // slot row of contraction row m: (b*E + e)*K + k with b = m / K; rows ascend by b_rstep, so (b, k) is
        // carried along instead of divided out per chunk
        int m = m_begin + i0 + b_r0;
        int b = m / p.K, k = m - b * p.K;
        for (int r = b_r0; r < KR; r += b_rstep) {
          const bool v = b_colvalid && (i0 + r < rows);
          const long long slot = static_cast<long long>(b * p.E + e) * p.K + k;
          f(stage_base + b_off + b_dst_seg + static_cast<uint32_t>(r) * 128u + swz(b_c, r),
            b_col + (v ? slot * row_bytes_d : 0ll), v, true);
          k += b_rstep;
          while (k >= p.K) { k -= p.K; ++b; }
        }
      } else {
        for (int idx = tid; idx < KR * cpr_b; idx += kProducerThreads) {
          const int r = idx / cpr_b, c = idx - r * cpr_b;
          const int m = m_begin + i0 + r;
          const long long goff = static_cast<long long>(g0) * ES + c * 16;
          const bool v = (i0 + r < rows) && goff < row_bytes_d;
          const char* src = Ys;
          if (v) {
            const int b = m / p.K, k = m - b * p.K;
            src = Ys + (static_cast<long long>(b * p.E + e) * p.K + k) * row_bytes_d + goff;
          }
          f(tile_addr<kMn32>(stage_base + b_off, seg_stride, r, c), src, v, true);
        }
      }
    };
    // Lean issue path for interior stages of full tiles (all KR rows inside this CTA's range with valid token
    // ids is not known statically, so rows keep their validity test; columns and the B walk are unpredicated).
    const bool a_cols_full = static_cast<long long>(f0) * ES + CPR_A * 16 <= row_bytes_g;
    const bool b_cols_full = b_fast && (KR % b_rstep == 0) && (b_rstep % 8 == 0 || kMn32) &&
                             (static_cast<long long>(g0) * ES + cpr_b * 16 <= row_bytes_d);
    const bool tile_full = a_cols_full && b_cols_full;
    const uint32_t a_dst0 = a_dst_seg + static_cast<uint32_t>(a_r0) * 128u + swz(a_c, a_r0);
    const uint32_t b_dst0 = b_dst_seg + static_cast<uint32_t>(b_r0) * 128u + swz(b_c, b_r0);
    const unsigned row_bytes_g32 = static_cast<unsigned>(row_bytes_g);
    // B source pointer of this thread's first row, carried across stages: rows ascend by b_rstep, a wrap of k
    // into the next batch element jumps (E-1)*K slot rows
    int bk = (m_begin + b_r0) % p.K;
    const char* b_ptr = b_col + (static_cast<long long>((m_begin + b_r0) / p.K * p.E + e) * p.K + bk) * row_bytes_d;
    const long long b_row_step = static_cast<long long>(b_rstep) * row_bytes_d;
    const long long b_wrap_step = static_cast<long long>(p.E - 1) * p.K * row_bytes_d;
    int b_next_kt = 0;     // the stage b_ptr currently points into
    auto issue_full = [&](int kt, uint32_t stage_base) {
      const int i0 = kt * KR;
      const uint32_t da = stage_base + a_dst0;
      // all table reads first: a copy instruction orders the memory accesses around it, so a look-up between
      // two copies would put its shared-memory latency on every copy
      constexpr int kIterA = KR / a_rstep;
      int tok[kIterA];
#pragma unroll
      for (int i = 0; i < kIterA; ++i) tok[i] = row_tok[i0 + a_r0 + i * a_rstep];
#pragma unroll
      for (int i = 0; i < kIterA; ++i) {
        const bool v = tok[i] >= 0;
        cp_async16(da + i * (a_rstep * 128u), a_col + static_cast<unsigned long long>(static_cast<unsigned>(v ? tok[i] : 0)) * row_bytes_g32,
                   v ? 16u : 0u);
      }
      const uint32_t db = stage_base + b_off + b_dst0;
      const uint32_t dstep = static_cast<uint32_t>(b_rstep) * 128u;
      const int iters = KR / b_rstep;
      for (int i = 0; i < iters; ++i) {
        cp_async16_full(db + i * dstep, b_ptr);
        b_ptr += b_row_step;
        bk += b_rstep;
        while (bk >= p.K) { bk -= p.K; b_ptr += b_wrap_step; }
      }
      b_next_kt = kt + 1;
    };
    const bool split_batched = STRICT && MT == 1 && KR / a_rstep <= 4 && b_fast && KR % b_rstep == 0 && KR / b_rstep <= 4;
    auto split_stage_batched = [&](int, uint32_t base) {
      uint32_t dst[8];
      bool on[8];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int ra = a_r0 + i * a_rstep, rb = b_r0 + i * b_rstep;
        dst[i] = base + a_dst_seg + static_cast<uint32_t>(ra) * 128u + swz(a_c, ra);
        on[i] = ra < KR;
        dst[4 + i] = base + b_off + b_dst_seg + static_cast<uint32_t>(rb) * 128u + swz(b_c, rb);
        on[4 + i] = rb < KR;
      }
      uint4 r[8];
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (on[i]) r[i] = lds16(dst[i]);
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (on[i]) split_store(dst[i], i < 4 ? a_lo_off : b_lo_off, r[i]);
    };
    auto issue_stage = [&](int kt, uint32_t base) {
      // the lean path walks b_ptr stage by stage, so it serves a prefix of consecutive full stages
      if (tile_full && kt == b_next_kt && (kt + 1) * KR <= rows) {
        issue_full(kt, base);
      } else {
        for_each_chunk(kt, base, true, [&](uint32_t dst, const char* src, bool v, bool) { cp_async16(dst, v ? src : Xs, v ? 16u : 0u); });
      }
    };
    bool alive;
    if (split_batched) alive = run_producer<STRICT>(pp, lane, issue_stage, split_stage_batched);
    else
    alive = run_producer<STRICT>(
        pp, lane,
        [&](int kt, uint32_t base) {
          // the lean path walks b_ptr stage by stage, so it serves a prefix of consecutive full stages
          if (tile_full && kt == b_next_kt && (kt + 1) * KR <= rows) {
            issue_full(kt, base);
          } else {
            for_each_chunk(kt, base, true, [&](uint32_t dst, const char* src, bool v, bool) { cp_async16(dst, v ? src : Xs, v ? 16u : 0u); });
          }
        },
        [&](int kc, uint32_t base) {
          for_each_chunk(kc, base, false, [&](uint32_t dst, const char*, bool, bool is_b) {
            split_chunk(dst, is_b ? b_lo_off : a_lo_off);
          });
        });

    // epilogue
    if (alive) {
      const int lg = warp & 3, half = warp >> 2;
      T* out = static_cast<T*>(p.out);
      if (p.out_layout == EGS_DW_GATHERED_ROWS) {
        // out[e, f, g]: rows f are contiguous over g -> transpose so that 8 lanes cover 128 bytes of one row
        const uint32_t tile = pp.tiles0 + static_cast<uint32_t>(warp) * 4096u;
        const int nblk = (bn + 31) >> 5;
        for (int mt = 0; mt < MT; ++mt)
        for (int c = half; c < nblk; c += 2) {
          const int gcol0 = g0 + c * 32;
          warp_block_emit(tmem_base + (static_cast<uint32_t>(lg * 32) << 16) + mt * acc_cols + static_cast<uint32_t>(c * 32), tile, lane,
                          pp.nk > 0, [&](int row, int cj, uint32_t x0, uint32_t x1, uint32_t x2, uint32_t x3) {
                            const int f = f0 + mt * kTileM + lg * 32 + row;
                            const int g = gcol0 + cj;
                            if (f < p.FG && g < p.FD) {
                              const long long off = (static_cast<long long>(e) * p.FG + f) * p.FD + g;
                              if (p.splits > 1) red4(p.acc + off, x0, x1, x2, x3);
                              else store4(out + off, x0, x1, x2, x3);
                            }
                          });
        }
      } else {
        // out[e, g, f]: for a fixed g consecutive lanes (f) are already contiguous in memory
        const int nch = bn >> 4;
        for (int mt = 0; mt < MT; ++mt)
        for (int c = half; c < nch; c += 2) {
          const int f = f0 + mt * kTileM + lg * 32 + lane;
          uint32_t v[16];
          if (pp.nk > 0) {
            tmem_ld16(tmem_base + (static_cast<uint32_t>(lg * 32) << 16) + mt * acc_cols + static_cast<uint32_t>(c * 16), v);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = 0u;
          }
          const int g = g0 + c * 16;
          const int nvalid = min(16, p.FD - g);
          if (f < p.FG && nvalid > 0) {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              if (i < nvalid) {
                const long long off = (static_cast<long long>(e) * p.FD + g + i) * p.FG + f;
                if (p.splits > 1) atomicAdd(p.acc + off, __uint_as_float(v[i]));
                else out[off] = from_f32<T>(__uint_as_float(v[i]));
              }
            }
          }
        }
      }
    }
  } else {
    if (lane == 0) {
      const uint32_t idesc = make_idesc(Elem<T>::fmt, 1u, 1u, kTileM, static_cast<uint32_t>(bn));
      const uint64_t k_adv = (UK * 128u) >> 4;
      run_mma_lane(pp, [&](int ks, uint32_t a_hi) {
        const uint32_t b_hi = a_hi + b_off;
        const int rrem = rows - ks * KR;
        const int nkq = min(KR / UK, (rrem + UK - 1) / UK);
        uint64_t ad = make_smem_desc(a_hi, seg_stride, kMnSbo, kMnLayout);
        uint64_t bd = make_smem_desc(b_hi, seg_stride, kMnSbo, kMnLayout);
        uint64_t adl = STRICT ? make_smem_desc(a_hi + a_lo_off, seg_stride, kMnSbo, kMnLayout) : 0ull;
        uint64_t bdl = STRICT ? make_smem_desc(b_hi + b_lo_off, seg_stride, kMnSbo, kMnLayout) : 0ull;
        // second accumulator (MT = 2): features 128..255 of the A tile, ES segments further on
        const uint64_t a_mt_adv = (static_cast<uint32_t>(ES) * seg_stride) >> 4;
        for (int kq = 0; kq < nkq; ++kq) {
          const uint32_t acc = (ks > 0 || kq > 0) ? 1u : 0u;
          if (STRICT) {
            umma<Elem<T>::tf32>(tmem_base, adl, bd, idesc, acc);
            umma<Elem<T>::tf32>(tmem_base, ad, bdl, idesc, 1u);
            umma<Elem<T>::tf32>(tmem_base, ad, bd, idesc, 1u);
          } else {
            umma<Elem<T>::tf32>(tmem_base, ad, bd, idesc, acc);
            if (MT == 2) umma<Elem<T>::tf32>(tmem_base + acc_cols, ad + a_mt_adv, bd, idesc, acc);
          }
          ad += k_adv; bd += k_adv; adl += k_adv; bdl += k_adv;
        }
      });
    }
    __syncwarp();
  }
  pipe_teardown(pp, tmem_base, tmem_cols, warp);
}

// ------------------------------------------------------------------------------------------------
// Fused pair  G -> S  for float32 tensors:   Mid = gather(Src) x W1[e]   (slot rows, stored),
//                                            Dst[token rows] += Mid x W2[e]
//   forward  : Src = X,    W1 = W_g, W2 = W_s (both EGS_W_CN)  ->  Mid = Y,  Dst = Out
//   backward : Src = dOut, W1 = W_s, W2 = W_g (both EGS_W_NC)  ->  Mid = dY, Dst = dX
// One CTA per (expert, 128 expert rows).  The 128 x N1 tile of Mid never leaves the SM between the two
// contractions: the epilogue warps read it from tensor memory, store it to global memory (the backward pass
// and the weight gradients need it) and write it into shared memory in the K-major swizzled operand format,
// from where the second contraction consumes it.  Saves one kernel launch per pair and the re-read of Mid -
// what the launch-latency-bound float32 configurations are made of.
//   warps 0..7   producers: stages of (gathered Src rows, W1 tile), then stages of W2 tiles, one ring
//   warps 8..15  epilogue : Mid tile (store + operand write), then the scatter epilogue (coalesced red.global.add)
//   warp  16     TMEM allocation; one lane issues all tcgen05.mma
// Conditions (checked on the host): float32, N1 a multiple of 32 and <= 256 (Mid rows are whole 128-byte
// segments), N2 <= one tile (128 strict / 256 TF32), row pitches multiples of 16 bytes.
// ------------------------------------------------------------------------------------------------
constexpr uint32_t kFusedHeaderBytes = 3072;
struct __align__(16) FusedHeader {
  unsigned long long full[kMaxStages];
  unsigned long long empty[kMaxStages];
  unsigned long long acc1_done, mid_ready, acc2_done, drain;
  uint32_t tmem_base;
  uint32_t abort_flag;
  int row_tok[kTileM];    // token row of every tile row (-1 = masked): gather source and scatter target
  int row_slot[kTileM];   // slot row of every tile row (-1 = beyond the expert's rows)
};
static_assert(sizeof(FusedHeader) <= kFusedHeaderBytes, "header does not fit");

template <bool STRICT>
__global__ void __launch_bounds__(17 * 32, 1) tensor_fused_pair_kernel(FusedParams p) {
  constexpr int ES = 4, KE = 32, UK = 8;          // float32: 32 elements per 128-byte segment, 8 per tcgen05.mma
  constexpr int kProdWarps = 8, kEpiWarps = 8, kProdThreads = kProdWarps * 32;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  FusedHeader* hdr = reinterpret_cast<FusedHeader*>(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int e = blockIdx.y;
  const int m0 = blockIdx.x * kTileM;
  const bool w_nc = (p.w_layout == EGS_W_NC);
  const int nseg_mid = p.N1 / KE;                                  // 128-byte segments per Mid row
  const uint32_t mid_bytes = static_cast<uint32_t>(nseg_mid) * kTileM * 128u;
  const uint32_t mid0 = smem_u32(smem_raw) + kFusedHeaderBytes;   // Mid operand tile (hi), then lo in strict mode
  const uint32_t mid_lo_off = mid_bytes;
  const uint32_t tiles0 = mid0 + mid_bytes * (STRICT ? 2u : 1u);  // stage ring
  // stage layouts: phase 1 = [A hi | A lo | B hi | B lo], phase 2 = [B hi | B lo]; one stage size for both
  const uint32_t a_bytes = kTileM * 128u;
  const int nseg_b1 = (p.BN1 * ES + 127) / 128, nseg_b2 = (p.BN2 * ES + 127) / 128;
  const uint32_t b1_bytes = w_nc ? static_cast<uint32_t>(p.BN1) * 128u : static_cast<uint32_t>(nseg_b1) * KE * 128u;
  const uint32_t b2_bytes = w_nc ? static_cast<uint32_t>(p.BN2) * 128u : static_cast<uint32_t>(nseg_b2) * KE * 128u;
  const uint32_t s1_bytes = (a_bytes + b1_bytes) * (STRICT ? 2u : 1u), s2_bytes = b2_bytes * (STRICT ? 2u : 1u);
  const uint32_t stage_bytes = s1_bytes > s2_bytes ? s1_bytes : s2_bytes;
  const uint32_t a_lo_off = a_bytes, b1_off = STRICT ? 2u * a_bytes : a_bytes, b1_lo_off = b1_bytes, b2_lo_off = b2_bytes;
  const int stages = p.stages;
  const int nk1 = (p.C1 + KE - 1) / KE, nk2 = nseg_mid;
  const uint32_t acc1_cols = tmem_cols_for(p.BN1), acc2_cols = tmem_cols_for(p.BN2);
  uint32_t tmem_cols = 32;
  while (tmem_cols < acc1_cols + acc2_cols) tmem_cols <<= 1;
  volatile uint32_t* abort_flag = &hdr->abort_flag;

  // ---- set-up ----
  if (tid < kTileM) {
    const int m = m0 + tid;
    int tok = -1, slot = -1;
    if (m < p.M) {
      const int b = m / p.K, k = m - b * p.K;
      slot = (b * p.E + e) * p.K + k;
      const long long t = load_index(p.Ind, p.index_dtype, slot);
      if (t >= 0 && t < p.T) tok = b * p.T + static_cast<int>(t);
      else if (p.status) atomicOr(p.status, EGS_STATUS_INDEX_OUT_OF_RANGE);
    }
    hdr->row_tok[tid] = tok;
    hdr->row_slot[tid] = slot;
  }
  if (tid == 0) {
    for (int s = 0; s < kMaxStages; ++s) {
      mbar_init(smem_u32(&hdr->full[s]), STRICT ? kProdWarps : kProdThreads);
      mbar_init(smem_u32(&hdr->empty[s]), 1);
    }
    mbar_init(smem_u32(&hdr->acc1_done), 1);
    mbar_init(smem_u32(&hdr->mid_ready), kEpiWarps);
    mbar_init(smem_u32(&hdr->acc2_done), 1);
    mbar_init(smem_u32(&hdr->drain), 1);
    fence_mbar_init();
    hdr->abort_flag = (p.status && (*reinterpret_cast<volatile int32_t*>(p.status) & EGS_STATUS_PIPELINE_TIMEOUT)) ? 1u : 0u;
    if (smem_misaligned(smem_raw)) {
      hdr->abort_flag = 1u;
      if (p.status) atomicOr(p.status, EGS_STATUS_INTERNAL);
    }
  }
  const int mma_warp = kProdWarps + kEpiWarps;
  if (warp == mma_warp) {
    tmem_alloc(smem_u32(&hdr->tmem_base), tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = hdr->tmem_base;
  const uint32_t acc1 = tmem_base, acc2 = tmem_base + acc1_cols;
  const bool run = (hdr->abort_flag == 0u);
  const int ntot = nk1 + nk2;
  if (!run) {
    // fall through to the common exit
  } else if (warp < kProdWarps) {
    // =========================== producers ===========================
    const char* Src = static_cast<const char*>(p.Src);
    const char* W1 = static_cast<const char*>(p.W1) + static_cast<long long>(e) * p.C1 * p.N1 * ES;
    const char* W2 = static_cast<const char*>(p.W2) + static_cast<long long>(e) * p.N1 * p.N2 * ES;
    const long long rb_src = static_cast<long long>(p.C1) * ES;    // row pitch of Src, and of W1 in NC layout
    const long long rb_n1 = static_cast<long long>(p.N1) * ES;     // row pitch of W1 in CN layout and of W2 in NC layout
    const long long rb_n2 = static_cast<long long>(p.N2) * ES;     // row pitch of W2 in CN layout
    const int cc = tid & 7, r0 = tid >> 3;
    const uint32_t rc_dst0 = static_cast<uint32_t>(r0) * 128u + (static_cast<uint32_t>(cc ^ (r0 & 7)) << 4);
    const char* a_src[kTileM / 32];
    uint32_t a_mask = 0;
#pragma unroll
    for (int i = 0; i < kTileM / 32; ++i) {
      const int tok = hdr->row_tok[r0 + 32 * i];
      a_src[i] = Src + (tok >= 0 ? static_cast<long long>(tok) * rb_src : 0ll) + cc * 16;
      if (tok >= 0) a_mask |= 1u << i;
    }
    const int cpr1 = nseg_b1 * 8, cpr2 = nseg_b2 * 8;
    // visits every 16-byte chunk this thread owns in stage g:  f(dst_hi_addr, src, valid, lo_offset)
    auto for_each_chunk = [&](int g, uint32_t base, auto&& f) {
      if (g < nk1) {
        const long long koff = static_cast<long long>(g) * 128;
        const bool kvalid = koff + cc * 16 < rb_src;
#pragma unroll
        for (int i = 0; i < kTileM / 32; ++i)
          f(base + rc_dst0 + i * 4096u, a_src[i] + koff, kvalid && ((a_mask >> i) & 1u), a_lo_off);
        if (w_nc) {       // W1 rows = n (N1 of them), contraction contiguous
          for (int r = r0; r < p.BN1; r += 32)
            f(base + b1_off + static_cast<uint32_t>(r) * 128u + (static_cast<uint32_t>(cc ^ (r & 7)) << 4),
              W1 + static_cast<long long>(r) * rb_src + koff + cc * 16, kvalid && r < p.N1, b1_lo_off);
        } else {          // W1 rows = contraction index, n contiguous
          for (int idx = tid; idx < KE * cpr1; idx += kProdThreads) {
            const int r = idx / cpr1, c = idx - r * cpr1;
            f(tile_addr<true>(base + b1_off, KE * 128u, r, c), W1 + static_cast<long long>(g * KE + r) * rb_n1 + c * 16,
              (g * KE + r) < p.C1 && c * 16 < rb_n1, b1_lo_off);
          }
        }
      } else {
        const int ks2 = g - nk1;
        if (w_nc) {       // W2 rows = n2, contraction (N1) contiguous
          const long long koff = static_cast<long long>(ks2) * 128;
          for (int r = r0; r < p.BN2; r += 32)
            f(base + static_cast<uint32_t>(r) * 128u + (static_cast<uint32_t>(cc ^ (r & 7)) << 4),
              W2 + static_cast<long long>(r) * rb_n1 + koff + cc * 16, r < p.N2, b2_lo_off);
        } else {          // W2 rows = contraction index (N1), n2 contiguous
          for (int idx = tid; idx < KE * cpr2; idx += kProdThreads) {
            const int r = idx / cpr2, c = idx - r * cpr2;
            f(tile_addr<true>(base, KE * 128u, r, c), W2 + static_cast<long long>(ks2 * KE + r) * rb_n2 + c * 16, c * 16 < rb_n2,
              b2_lo_off);
          }
        }
      }
    };
    auto issue = [&](int g, uint32_t base) {
      for_each_chunk(g, base, [&](uint32_t dst, const char* src, bool v, uint32_t) { cp_async16(dst, v ? src : Src, v ? 16u : 0u); });
    };
    bool alive = true;
    if (!STRICT) {
      for (int g = 0; g < ntot; ++g) {
        const int slot = g % stages, use = g / stages;
        if (use > 0) alive = mbar_wait_warp(smem_u32(&hdr->empty[slot]), (use - 1) & 1, abort_flag, p.status, lane);
        if (!alive) break;
        issue(g, tiles0 + slot * stage_bytes);
        cp_async_mbar_arrive_noinc(smem_u32(&hdr->full[slot]));
      }
    } else {
      const int dist = stages - 1;
      for (int g = 0; g < dist; ++g) {
        if (g < ntot) issue(g, tiles0 + (g % stages) * stage_bytes);
        cp_async_commit();
      }
      for (int gc = 0; gc < ntot; ++gc) {
        cp_async_wait_pending(dist - 1);
        if (alive) {
          for_each_chunk(gc, tiles0 + (gc % stages) * stage_bytes,
                         [&](uint32_t dst, const char*, bool, uint32_t lo_off) { split_store(dst, lo_off, lds16(dst)); });
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&hdr->full[gc % stages]));
        }
        const int g = gc + dist;
        if (g < ntot && alive) {
          const int use = g / stages;
          if (use > 0) alive = mbar_wait_warp(smem_u32(&hdr->empty[g % stages]), (use - 1) & 1, abort_flag, p.status, lane);
          if (alive) issue(g, tiles0 + (g % stages) * stage_bytes);
        }
        cp_async_commit();
      }
    }
    cp_async_wait_all();
  } else if (warp < kProdWarps + kEpiWarps) {
    // =========================== epilogue warps ===========================
    const int ew = warp - kProdWarps;
    const int lg = ew & 3, half = ew >> 2;        // TMEM lane group (= warp index modulo 4), half of the column blocks
    const int row = lg * 32 + lane;               // tile row this thread owns in tensor memory
    const uint32_t lane_base = static_cast<uint32_t>(lg * 32) << 16;
    bool alive = true;
    if (nk1 > 0) alive = mbar_wait_warp(smem_u32(&hdr->acc1_done), 0u, abort_flag, p.status, lane);
    if (alive) {
      tc_fence_after();
      // (1) Mid tile: tensor memory -> shared memory in the K-major operand format (segment = 32 columns)
      for (int c = half; c < nseg_mid; c += 2) {
        uint32_t v[32];
        if (nk1 > 0) {
          tmem_ld32(acc1 + lane_base + static_cast<uint32_t>(c * 32), v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0u;
        }
        const uint32_t seg = mid0 + static_cast<uint32_t>(c) * (kTileM * 128u) + static_cast<uint32_t>(row) * 128u;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint32_t addr = seg + (static_cast<uint32_t>(j ^ (row & 7)) << 4);
          const uint4 x = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
          asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(x.x), "r"(x.y), "r"(x.z), "r"(x.w) : "memory");
          if (STRICT) split_store(addr, mid_lo_off, x);
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&hdr->mid_ready));
      // (2) the same rows go to global memory, read back from the tile so that 8 lanes cover 128 contiguous bytes
      float* mid_out = static_cast<float*>(p.Mid);
      const int j = lane & 7;
      for (int c = half; c < nseg_mid; c += 2) {
        const uint32_t seg = mid0 + static_cast<uint32_t>(c) * (kTileM * 128u);
        uint4 x[8];
#pragma unroll
        for (int it = 0; it < 8; ++it) {
          const int r = lg * 32 + it * 4 + (lane >> 3);
          x[it] = lds16(seg + static_cast<uint32_t>(r) * 128u + (static_cast<uint32_t>(j ^ (r & 7)) << 4));
        }
#pragma unroll
        for (int it = 0; it < 8; ++it) {
          const int r = lg * 32 + it * 4 + (lane >> 3);
          const int slot = hdr->row_slot[r];
          if (slot >= 0) *reinterpret_cast<uint4*>(mid_out + static_cast<long long>(slot) * p.N1 + c * 32 + j * 4) = x[it];
        }
      }
      // (3) scatter epilogue: the stage ring is idle once acc2_done has completed; its first 32 KB are the
      //     warps' transpose tiles
      alive = mbar_wait_warp(smem_u32(&hdr->acc2_done), 0u, abort_flag, p.status, lane);
      if (alive) {
        tc_fence_after();
        const uint32_t tile = tiles0 + static_cast<uint32_t>(ew) * 4096u;
        const int nblk = (p.BN2 + 31) >> 5;
        for (int c = half; c < nblk; c += 2) {
          warp_block_emit(acc2 + lane_base + static_cast<uint32_t>(c * 32), tile, lane, true,
                          [&](int r, int cj, uint32_t x0, uint32_t x1, uint32_t x2, uint32_t x3) {
                            const int tok = hdr->row_tok[lg * 32 + r];
                            const int col = c * 32 + cj;
                            if (tok >= 0 && col < p.N2) red4(p.Dst + static_cast<long long>(tok) * p.N2 + col, x0, x1, x2, x3);
                          });
        }
      }
    }
  } else {
    // =========================== MMA issuer ===========================
    if (lane == 0) {
      const uint32_t b_lbo = w_nc ? 16u : KE * 128u;
      const uint32_t b_sbo = w_nc ? 1024u : 512u;
      const uint32_t b_lay = w_nc ? kSwizzle128 : kSwizzle128Base32;
      const uint64_t a_adv = 32u >> 4, b_adv = (w_nc ? 32u : UK * 128u) >> 4;
      const uint32_t idesc1 = make_idesc(2u, 0u, w_nc ? 0u : 1u, kTileM, static_cast<uint32_t>(p.BN1));
      const uint32_t idesc2 = make_idesc(2u, 0u, w_nc ? 0u : 1u, kTileM, static_cast<uint32_t>(p.BN2));
      bool ok = true;
      for (int g = 0; g < ntot && ok; ++g) {
        const int slot = g % stages;
        if (g == nk1) {
          // the Mid operand tile must be complete before the second contraction starts
          ok = mbar_wait(smem_u32(&hdr->mid_ready), 0u, abort_flag, p.status);
          if (!ok) break;
        }
        ok = mbar_wait(smem_u32(&hdr->full[slot]), (g / stages) & 1, abort_flag, p.status);
        if (!ok) break;
        tc_fence_after();
        const uint32_t base = tiles0 + slot * stage_bytes;
        const bool ph1 = g < nk1;
        const int ks = ph1 ? g : g - nk1;
        const uint32_t a_hi = ph1 ? base : mid0 + static_cast<uint32_t>(ks) * (kTileM * 128u);
        const uint32_t a_lo = ph1 ? base + a_lo_off : a_hi + mid_lo_off;
        const uint32_t b_hi = ph1 ? base + b1_off : base;
        const uint32_t b_lo = b_hi + (ph1 ? b1_lo_off : b2_lo_off);
        const int krem = ph1 ? p.C1 - ks * KE : KE;
        const int nkq = min(KE / UK, (krem + UK - 1) / UK);
        uint64_t ad = make_smem_desc(a_hi, 16u, 1024u);
        uint64_t adl = STRICT ? make_smem_desc(a_lo, 16u, 1024u) : 0ull;
        uint64_t bd = make_smem_desc(b_hi, b_lbo, b_sbo, b_lay);
        uint64_t bdl = STRICT ? make_smem_desc(b_lo, b_lbo, b_sbo, b_lay) : 0ull;
        const uint32_t d = ph1 ? acc1 : acc2;
        const uint32_t idesc = ph1 ? idesc1 : idesc2;
        for (int kq = 0; kq < nkq; ++kq) {
          const uint32_t acc = (ks > 0 || kq > 0) ? 1u : 0u;
          if (STRICT) {
            umma<true>(d, adl, bd, idesc, acc);
            umma<true>(d, ad, bdl, idesc, 1u);
            umma<true>(d, ad, bd, idesc, 1u);
          } else {
            umma<true>(d, ad, bd, idesc, acc);
          }
          ad += a_adv;
          adl += a_adv;
          bd += b_adv;
          bdl += b_adv;
        }
        umma_commit(smem_u32(&hdr->empty[slot]));
        if (g == nk1 - 1) umma_commit(smem_u32(&hdr->acc1_done));
        if (g == ntot - 1) umma_commit(smem_u32(&hdr->acc2_done));
      }
    }
    __syncwarp();
  }

  // ---- common exit ----
  tc_fence_before();
  __syncthreads();
  if (warp == mma_warp) tmem_release(tmem_base, tmem_cols, smem_u32(&hdr->drain), abort_flag, lane);
}

// ------------------------------------------------------------------------------------------------
// Self-test of the bounded wait: one CTA waits on an mbarrier that nobody ever completes, with a short limit.
// The wait must give up, raise the abort flag and EGS_STATUS_PIPELINE_TIMEOUT, and the kernel must return normally
// (the context stays usable).  out[0] = 1 if the wait returned false, out[1] = the abort flag afterwards.
// ------------------------------------------------------------------------------------------------
__global__ void wait_timeout_selftest_kernel(int32_t* status, int* out, long long limit_cycles) {
  __shared__ __align__(8) unsigned long long bar;
  __shared__ uint32_t abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    fence_mbar_init();
    abort_flag = 0u;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const bool ok = mbar_wait(smem_u32(&bar), 0u, &abort_flag, status, limit_cycles);
    out[0] = ok ? 0 : 1;
    out[1] = static_cast<int>(abort_flag);
  }
}

// ------------------------------------------------------------------------------------------------
// host side: tile / stage selection and launches
// ------------------------------------------------------------------------------------------------
constexpr size_t kSmemPerSm = 228 * 1024;
constexpr size_t kSmemReservedPerCta = 1024;
constexpr size_t kSmemMaxPerCta = 227 * 1024;
constexpr int kSmCount = 148;


// Pipeline depth: large grids aim at two CTAs per SM (the prologue and epilogue of one CTA overlap the main
// loop of the other); grids that fit in one wave take the whole SM.
int pick_stages(size_t fixed_bytes, size_t stage_bytes, long long ctas, bool allow_two_per_sm) {
  const size_t two = kSmemPerSm / 2 - kSmemReservedPerCta;
  int s = 0;
  if (allow_two_per_sm && ctas > kSmCount && fixed_bytes + 2 * stage_bytes <= two)
    s = static_cast<int>((two - fixed_bytes) / stage_bytes);
  else
    s = static_cast<int>((kSmemMaxPerCta - fixed_bytes) / stage_bytes);
  if (s > kMaxStages) s = kMaxStages;
  return s;
}

}  // namespace

size_t configure_tensor_rowgemm(RowGemmParams& p, bool scatter, int dtype, int precision) {
  const int es = (dtype == EGS_F32) ? 4 : 2;
  const bool strict = (dtype == EGS_F32 && precision == EGS_PREC_STRICT);
  const int ke = 128 / es;
  int bn = (p.N + 15) & ~15;
  const int cap = strict ? 128 : 256;
  if (bn > cap) bn = cap;
  // strict float32 doubles every tile (hi + lo): when the grid is larger than one wave, 64-wide tiles keep a
  // 2-stage ring under half an SM's shared memory so that two CTAs share an SM
  if (strict && bn > 64 &&
      static_cast<long long>((p.M + kTileM - 1) / kTileM) * ((p.N + bn - 1) / bn) * p.E > kSmCount)
    bn = 64;
  p.BN = bn;
  const size_t nseg_b = (static_cast<size_t>(bn) * es + 127) / 128;
  const size_t b_bytes = (p.w_layout == EGS_W_NC) ? static_cast<size_t>(bn) * 128 : nseg_b * ke * 128;
  const size_t fixed = kHeaderBytes;
  const long long n_tiles = (p.N + bn - 1) / bn;
  // 256-row CTAs (two accumulators): when the grid still fills the SMs at least once, the contraction is long
  // enough for the deeper ring to matter, and the two accumulators fit in tensor memory
  const long long ctas2 = static_cast<long long>((p.M + 2 * kTileM - 1) / (2 * kTileM)) * n_tiles * p.E;
  // (the scatter epilogue dominates short contractions and profits from two CTAs per SM instead)
  const bool want2 = !strict && p.M >= 2 * kTileM && ctas2 >= kSmCount && p.C * es >= (scatter ? 4096 : 1024);
  p.row_tiles = want2 ? 2 : 1;
  const size_t a_bytes = static_cast<size_t>(kTileM) * p.row_tiles * 128;
  const size_t stage_bytes = (a_bytes + b_bytes) * (strict ? 2 : 1);
  const long long ctas = static_cast<long long>((p.M + kTileM * p.row_tiles - 1) / (kTileM * p.row_tiles)) * n_tiles * p.E;
  // persistent variant (see its kernel): scatter problems with many tiles, non-strict arithmetic
  const long long tiles1 = static_cast<long long>((p.M + kTileM - 1) / kTileM) * n_tiles * p.E;
  p.persistent = 0;
  // direct 16-bit scatter adds go out as bulk reductions
  p.bulk_epilogue = (scatter && es == 2) ? 1 : 0;
  // (measured: it wins for contractions of up to four stages - the scatter of cfg4 and cfg2 - and loses for longer ones)
  if (!strict && scatter && p.C * es <= 512 && tiles1 >= 2 * kSmCount) {
    const size_t st1 = static_cast<size_t>(kTileM) * 128 + b_bytes;
    size_t fixed_p = kPersistHeaderBytes + kPersistMaxEpilogueWarps * 4096;
    // 16-bit scatter: staging buffers for the bulk adds when the ring keeps three stages
    const size_t bulk_bytes = (kPersistMaxEpilogueWarps * 2 * kBulkBufBytes + 1023) & ~static_cast<size_t>(1023);
    const bool bulk_fits = (kSmemMaxPerCta - kPersistHeaderBytes - bulk_bytes) / st1 >= 3;
    if (p.bulk_epilogue && bulk_fits) fixed_p = kPersistHeaderBytes + bulk_bytes;
    size_t ns = (kSmemMaxPerCta - fixed_p) / st1;
    if (ns > static_cast<size_t>(kMaxStages)) ns = kMaxStages;
    if (ns >= 3) {
      p.persistent = 1;
      p.row_tiles = 1;
      p.stages = static_cast<int>(ns);
      if (!bulk_fits) p.bulk_epilogue = 0;
      return fixed_p + ns * st1;
    }
  }
  p.stages = pick_stages(fixed, stage_bytes, ctas, p.row_tiles == 1);
  return fixed + p.stages * stage_bytes;
}

size_t configure_tensor_dweight(DWeightParams& p, int dtype, int precision) {
  const int es = (dtype == EGS_F32) ? 4 : 2;
  const bool strict = (dtype == EGS_F32 && precision == EGS_PREC_STRICT);
  const int kr = 128 / es;
  int bn = (p.FD + 15) & ~15;
  const int cap = strict ? 64 : 256;   // strict: 64-wide tiles so that two CTAs share an SM
  if (bn > cap) bn = cap;
  p.BN = bn;
  const size_t seg_stride = static_cast<size_t>(kr) * 128;
  const size_t nseg_b = (static_cast<size_t>(bn) * es + 127) / 128;
  // 256-feature CTAs (two accumulators): long contractions whose grid still covers the SMs, non-strict only
  const long long tiles2 = static_cast<long long>((p.FG + 2 * kTileM - 1) / (2 * kTileM)) * ((p.FD + bn - 1) / bn) * p.E;
  const bool want2 = !strict && p.FG > kTileM && tiles2 >= kSmCount && p.M >= 16 * kr && bn * 2 <= 512;
  p.row_tiles = want2 ? 2 : 1;
  const size_t a_bytes = es * seg_stride * p.row_tiles;
  const size_t stage_bytes = (a_bytes + nseg_b * seg_stride) * (strict ? 2 : 1);
  // split the contraction so that the grid fills one wave of CTAs and no CTA owns more rows than the
  // shared-memory row table holds
  const int f_tile = kTileM * p.row_tiles;
  const long long tiles = static_cast<long long>((p.FG + f_tile - 1) / f_tile) * ((p.FD + bn - 1) / bn) * p.E;
  // as many row ranges as still fit in one wave of CTAs (two CTAs per SM with 128-feature tiles)
  long long want = (static_cast<long long>(kSmCount) * (p.row_tiles == 2 ? 1 : 2)) / tiles;
  // Strict float32: the tensor core adds every product group into the float32 accumulator with truncation, an error that
  // grows with the number of accumulation steps (measured 1.5e-5 of max|ref| after 8192 contraction rows, against a
  // 1e-5 bar).  Ranges of at most 1024 rows keep it near 3e-6; the partial tiles are then summed by float32 atomics,
  // which round correctly.
  const int max_rows = strict ? 1024 : kMaxRowsPerSplit;
  const long long min_splits = (p.M + max_rows - 1) / max_rows;
  if (want < min_splits) want = min_splits;
  const long long max_splits = (p.M + kr - 1) / kr;
  if (want > max_splits) want = max_splits;
  if (want < 1) want = 1;
  long long rows = (p.M + want - 1) / want;
  rows = (rows + kr - 1) / kr * kr;
  if (rows < kr) rows = kr;
  p.rows_per_split = static_cast<int>(rows);
  p.splits = static_cast<int>((p.M + rows - 1) / rows);
  if (p.splits < 1) p.splits = 1;
  const size_t table_bytes = (static_cast<size_t>(rows) * 4 + 1023) & ~static_cast<size_t>(1023);
  const size_t fixed = kHeaderBytesD + table_bytes;
  p.stages = pick_stages(fixed, stage_bytes, tiles * p.splits, p.row_tiles == 1);
  return fixed + p.stages * stage_bytes;
}

size_t configure_tensor_fused_pair(FusedParams& p, int precision) {
  const bool strict = (precision == EGS_PREC_STRICT);
  const size_t es = 4, ke = 32;
  if (p.C1 < 1 || p.C1 % 4 != 0 || p.N2 < 1 || p.N2 % 4 != 0) return 0;    // 16-byte row pitches
  if (p.N1 < 32 || p.N1 > 256 || p.N1 % 32 != 0) return 0;                 // Mid rows are whole 128-byte segments
  const int bn2 = (p.N2 + 15) & ~15;
  if (bn2 > (strict ? 128 : 256)) return 0;                                // one tile over N2
  p.BN1 = p.N1;
  p.BN2 = bn2;
  const bool nc = (p.w_layout == EGS_W_NC);
  const size_t a_bytes = static_cast<size_t>(kTileM) * 128;
  const size_t nseg1 = (p.BN1 * es + 127) / 128, nseg2 = (p.BN2 * es + 127) / 128;
  const size_t b1 = nc ? static_cast<size_t>(p.BN1) * 128 : nseg1 * ke * 128;
  const size_t b2 = nc ? static_cast<size_t>(p.BN2) * 128 : nseg2 * ke * 128;
  const size_t s1 = (a_bytes + b1) * (strict ? 2 : 1), s2 = b2 * (strict ? 2 : 1);
  const size_t stage_bytes = s1 > s2 ? s1 : s2;
  const size_t mid = static_cast<size_t>(p.N1 / 32) * kTileM * 128 * (strict ? 2 : 1);
  const size_t fixed = kFusedHeaderBytes + mid;
  if (fixed + 2 * stage_bytes > kSmemMaxPerCta) return 0;
  size_t ns = (kSmemMaxPerCta - fixed) / stage_bytes;
  const size_t ntot = static_cast<size_t>((p.C1 + 31) / 32 + p.N1 / 32);
  if (ns > ntot) ns = ntot;
  if (ns > static_cast<size_t>(kMaxStages)) ns = kMaxStages;
  if (ns < 2 || ns * stage_bytes < 8u * 4096u) return 0;                   // the ring doubles as the transpose tiles
  p.stages = static_cast<int>(ns);
  return fixed + ns * stage_bytes;
}

// The opt-in to large dynamic shared memory is per kernel function: done once, for the maximum.
template <auto kernel>
static cudaError_t ensure_smem_optin() {
  static thread_local int done_device = -1;
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  if (done_device == dev) return cudaSuccess;
  err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kSmemMaxPerCta));
  if (err == cudaSuccess) done_device = dev;
  return err;
}

cudaError_t launch_tensor_rowgemm(const RowGemmParams& p, bool scatter, int dtype, int precision, size_t smem_bytes,
                                  cudaStream_t st) {
  if (p.persistent) {
    const int row_blocks = p.E * ((p.M + kTileM - 1) / kTileM);
    dim3 pgrid(row_blocks < kSmCount ? row_blocks : kSmCount);
    dim3 pblock(scatter ? PersistShape<true>::kThreads : PersistShape<false>::kThreads);
    cudaError_t perr = cudaSuccess;
#define EGS_LAUNCH_P(TY)                                                                                     \
  do {                                                                                                       \
    if (scatter) {                                                                                           \
      perr = (ensure_smem_optin<tensor_rowgemm_persistent_kernel<TY, true>>());                              \
      if (perr == cudaSuccess) tensor_rowgemm_persistent_kernel<TY, true><<<pgrid, pblock, smem_bytes, st>>>(p);  \
    } else {                                                                                                 \
      perr = (ensure_smem_optin<tensor_rowgemm_persistent_kernel<TY, false>>());                             \
      if (perr == cudaSuccess) tensor_rowgemm_persistent_kernel<TY, false><<<pgrid, pblock, smem_bytes, st>>>(p); \
    }                                                                                                        \
  } while (0)
    if (dtype == EGS_F32) EGS_LAUNCH_P(float);
    else if (dtype == EGS_F16) EGS_LAUNCH_P(__half);
    else EGS_LAUNCH_P(__nv_bfloat16);
#undef EGS_LAUNCH_P
    if (perr != cudaSuccess) return perr;
    count_launch();
    return cudaGetLastError();
  }
  const int rows_per_cta = kTileM * p.row_tiles;
  const int row_tiles = (p.M + rows_per_cta - 1) / rows_per_cta;
  dim3 grid(p.expert_fastest ? p.E : row_tiles, (p.N + p.BN - 1) / p.BN, p.expert_fastest ? row_tiles : p.E);
  dim3 block(kThreads);
  cudaError_t err = cudaSuccess;
#define EGS_LAUNCH2(TY, STRICT, SC, MTV)                                                              \
  do {                                                                                                \
    err = (ensure_smem_optin<tensor_rowgemm_kernel<TY, STRICT, SC, MTV>>());                          \
    if (err == cudaSuccess) tensor_rowgemm_kernel<TY, STRICT, SC, MTV><<<grid, block, smem_bytes, st>>>(p); \
  } while (0)
#define EGS_LAUNCH(TY, STRICT)                                        \
  do {                                                                \
    if (scatter) {                                                    \
      if (p.row_tiles == 2 && !STRICT) EGS_LAUNCH2(TY, false, true, 2);  \
      else EGS_LAUNCH2(TY, STRICT, true, 1);                          \
    } else {                                                          \
      if (p.row_tiles == 2 && !STRICT) EGS_LAUNCH2(TY, false, false, 2); \
      else EGS_LAUNCH2(TY, STRICT, false, 1);                         \
    }                                                                 \
  } while (0)
  if (dtype == EGS_F32) {
    if (precision == EGS_PREC_STRICT) EGS_LAUNCH(float, true);
    else EGS_LAUNCH(float, false);
  } else if (dtype == EGS_F16) {
    EGS_LAUNCH(__half, false);
  } else {
    EGS_LAUNCH(__nv_bfloat16, false);
  }
#undef EGS_LAUNCH
#undef EGS_LAUNCH2
  if (err != cudaSuccess) return err;
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_tensor_dweight(const DWeightParams& p, int dtype, int precision, size_t smem_bytes, cudaStream_t st) {
  const int f_tile = kTileM * p.row_tiles;
  dim3 grid((p.FG + f_tile - 1) / f_tile, (p.FD + p.BN - 1) / p.BN, p.E * p.splits);
  dim3 block(kThreads);
  cudaError_t err = cudaSuccess;
#define EGS_LAUNCH_D(TY, STRICT, MTV)                                                           \
  do {                                                                                          \
    err = (ensure_smem_optin<tensor_dweight_kernel<TY, STRICT, MTV>>());                        \
    if (err == cudaSuccess) tensor_dweight_kernel<TY, STRICT, MTV><<<grid, block, smem_bytes, st>>>(p); \
  } while (0)
#define EGS_LAUNCH(TY, STRICT)                                   \
  do {                                                           \
    if (p.row_tiles == 2 && !STRICT) EGS_LAUNCH_D(TY, false, 2); \
    else EGS_LAUNCH_D(TY, STRICT, 1);                            \
  } while (0)
  if (dtype == EGS_F32) {
    if (precision == EGS_PREC_STRICT) EGS_LAUNCH(float, true);
    else EGS_LAUNCH(float, false);
  } else if (dtype == EGS_F16) {
    EGS_LAUNCH(__half, false);
  } else {
    EGS_LAUNCH(__nv_bfloat16, false);
  }
#undef EGS_LAUNCH
#undef EGS_LAUNCH_D
  if (err != cudaSuccess) return err;
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_wait_timeout_selftest(int32_t* status, int* out, long long limit_cycles, cudaStream_t st) {
  wait_timeout_selftest_kernel<<<1, 32, 0, st>>>(status, out, limit_cycles);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_tensor_fused_pair(const FusedParams& p, int precision, size_t smem_bytes, cudaStream_t st) {
  dim3 grid((p.M + kTileM - 1) / kTileM, p.E);
  dim3 block(17 * 32);
  cudaError_t err;
  if (precision == EGS_PREC_STRICT) {
    err = ensure_smem_optin<tensor_fused_pair_kernel<true>>();
    if (err == cudaSuccess) tensor_fused_pair_kernel<true><<<grid, block, smem_bytes, st>>>(p);
  } else {
    err = ensure_smem_optin<tensor_fused_pair_kernel<false>>();
    if (err == cudaSuccess) tensor_fused_pair_kernel<false><<<grid, block, smem_bytes, st>>>(p);
  }
  if (err != cudaSuccess) return err;
  count_launch();
  return cudaGetLastError();
}

}  // namespace egs

