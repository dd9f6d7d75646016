// Fused pair  G -> S  for 16-bit tensors (bf16 / fp16), persistent, sm_100a only:
//     Mid = gather(Src) x W1[e]            (slot rows, stored: the backward pass and the weight gradients read them)
//     Dst[token rows] += Mid x W2[e]
//   forward  : Src = X,    W1 = W_g, W2 = W_s (both EGS_W_CN)  ->  Mid = Y,  Dst = Out
//   backward : Src = dOut, W1 = W_s, W2 = W_g (both EGS_W_NC)  ->  Mid = dY, Dst = dX
//
// Why one kernel: a scatter kernel alone leaves the tensor core idle while its epilogue drains, and a gather kernel
// alone writes Mid only for the scatter to read it back.  Here the gather contraction of the NEXT row block runs under
// the scatter epilogue of the current one, and Mid reaches the second contraction through tensor memory.
//
// One CTA per SM walks (expert, 128 expert rows) row blocks.  Per row block t:
//   G(t)   acc1[128 x N1]  = gathered Src rows x W1[e]          (contraction C1 in stages of 64 elements)
//   conv   Y(t) = acc1 rounded to 16 bits: written to tensor memory as the A operand of the second contraction
//          (lane = row, two elements per 32-bit column) and stored to global memory
//   S(t)   for every 64-wide tile nt of N2:  acc2[nt & 1][128 x 64] = Y(t) x W2[e][:, tile]  (A from tensor memory,
//          whole contraction N1 in one stage), then the scatter epilogue adds the tile to the token rows
// The stages go through ONE ring in a fixed order - S(t,0), G(t+1,0), S(t,1), G(t+1,1), ... - so that the gather
// contraction of the next row block is spread under the scatter epilogue of this one.
//   warps 0..7    producers: 16-byte cp.async gathers of the Src rows; one thread issues the TMA loads of the W tiles
//   warps 8..11   converters: acc1 -> Y (tensor memory + global store)
//   warps 12..19  scatter epilogue, two groups of four warps (one per TMEM lane group) taking pairs of S tiles in turn:
//                 acc2 -> 16 bits -> staged in shared memory -> one bulk reduction per row and tile pair into the output
//                 rows; or (heavy collisions, decided by the planning flag) float32 red.global.add into the rows of the scratch
//   warp  20      TMEM allocation; one lane issues the tcgen05.mma of the G stages
//   warp  21      one lane issues the tcgen05.mma of the S tiles
// Tensor memory (512 columns): Y [0,128), acc1 [128,384), acc2[0] [384,448), acc2[1] [448,512).
// What paces the roles is instruction latency, not bandwidth: a lone lane executes about one instruction per 7-10
// clocks, and a hand-over through an mbarrier costs several hundred.  Hence: two issuing lanes (each walks the ring order
// and skips the other's stages), tcgen05.mma issued in straight-line groups, both S accumulators in flight so that no
// role waits for a round trip, no divisions on the per-stage paths, W tiles by TMA instead of 16-byte copies.
// Every wait is bounded; when one runs out the CTA raises its abort flag and EGS_STATUS_PIPELINE_TIMEOUT and all roles
// fall through to the common exit.
#include "egs_tcgen05.cuh"

namespace egs {

namespace {

constexpr int kP16ProducerWarps = 8;
constexpr int kP16ConvertWarps = 4;
constexpr int kP16ScatterWarps = 8;                          // two groups of four
constexpr int kP16ProducerThreads = kP16ProducerWarps * 32;
constexpr int kP16WarpG = kP16ProducerWarps + kP16ConvertWarps + kP16ScatterWarps;   // issues the G stages, owns TMEM
constexpr int kP16WarpS = kP16WarpG + 1;                                             // issues the S tiles
constexpr int kP16Threads = (kP16WarpS + 1) * 32;
constexpr int kP16NT = 64;                                   // scatter tile width: one 128-byte segment of 16-bit elements
constexpr uint32_t kP16HeaderBytes = 1024;
constexpr uint32_t kP16RowPitch = 2u * kP16NT * 2u + 16u;    // two tiles staged side by side + 16: conflict-free 16-byte stores
constexpr uint32_t kP16BufBytes = 32u * kP16RowPitch;        // one 32-row staging buffer
constexpr uint32_t kP16StagingBytes = kP16ScatterWarps * kP16BufBytes;        // one staging buffer per scatter warp
constexpr uint32_t kP16RingOffset = (kP16HeaderBytes + kP16StagingBytes + 1023u) & ~1023u;
constexpr uint32_t kP16ColY = 0, kP16ColAcc1 = 128, kP16ColAcc2 = 384, kP16TmemCols = 512;
static_assert(4096u <= kP16BufBytes, "the float32 transpose tile fits in a warp's staging area");

struct __align__(16) P16Header {
  unsigned long long full[kMaxStages];
  unsigned long long empty[kMaxStages];
  unsigned long long acc1_full, y_ready, s_done;
  unsigned long long acc2_full[4];    // [2 * group + buffer]: a tile for scatter group `group` is complete in acc2[buffer]
  unsigned long long acc2_empty[2];   // [buffer]: the tile in acc2[buffer] has been read
  unsigned long long drain;
  uint32_t tmem_base;
  uint32_t abort_flag;
};
static_assert(sizeof(P16Header) <= kP16HeaderBytes, "header does not fit");

__device__ __forceinline__ void bulk_wait_read_0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }

struct P16Block {
  int e, m0;
};
__device__ __forceinline__ P16Block p16_block(const FusedParams& p, int rb, int m_tiles) {
  P16Block r;
  if (p.expert_fastest) {
    r.e = rb % p.E;
    r.m0 = (rb / p.E) * kTileM;
  } else {
    r.m0 = (rb % m_tiles) * kTileM;
    r.e = rb / m_tiles;
  }
  return r;
}
// Token row (gather source and scatter target) and slot row of expert row m of expert e; -1 = masked.
__device__ __forceinline__ void p16_rows(const FusedParams& p, int e, int m, int& tok, int& slot, bool report) {
  tok = -1;
  slot = -1;
  if (m >= p.M) return;
  const int b = m / p.K, k = m - b * p.K;
  slot = (b * p.E + e) * p.K + k;
  const long long t = load_index(p.Ind, p.index_dtype, slot);
  if (t >= 0 && t < p.T) tok = b * p.T + static_cast<int>(t);
  else if (report && p.status) atomicOr(p.status, EGS_STATUS_INDEX_OUT_OF_RANGE);
}

// Position in the stage ring; advanced once per stage by every role that follows the ring order.
struct P16Ring {
  int slot = 0;
  uint32_t round = 0;
  __device__ __forceinline__ void advance(int stages) {
    if (++slot == stages) {
      slot = 0;
      ++round;
    }
  }
};

template <typename T>
__global__ void __launch_bounds__(kP16Threads, 1) tensor_pair16_persistent_kernel(FusedParams p, const __grid_constant__ TensorMap3 map_w1,
                                                                                  const __grid_constant__ TensorMap3 map_w2) {
  constexpr int ES = 2, KE = 64, UK = 16;       // 64 contraction elements per G stage, 16 per tcgen05.mma
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  P16Header* hdr = reinterpret_cast<P16Header*>(smem_raw);
  const uint32_t smem0 = smem_u32(smem_raw);
  const uint32_t staging0 = smem0 + kP16HeaderBytes;
  const uint32_t ring0 = smem0 + kP16RingOffset;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool w_nc = (p.w_layout == EGS_W_NC);
  const int m_tiles = (p.M + kTileM - 1) / kTileM;
  const int row_blocks = p.E * m_tiles;
  const int nk1 = (p.C1 + KE - 1) / KE;                  // G stages per row block
  const int n2 = (p.N2 + kP16NT - 1) / kP16NT;           // S tiles (= S stages) per row block
  const int steps = nk1 > n2 ? nk1 : n2;                 // interleaving steps per row block: S(t,i) then G(t+1,i)
  const int stages = p.stages;
  const uint32_t slot_bytes = p.slot_bytes;
  const uint32_t a_bytes = kTileM * 128u;
  const int nseg_b1 = (p.BN1 * ES + 127) / 128;          // 128-byte segment columns of a W1 tile in CN layout
  const int nseg_b2 = (p.N1 * ES + 127) / 128;           // 128-byte contraction segments of a W2 tile in NC layout
  volatile uint32_t* abort_flag = &hdr->abort_flag;

  // ---- set-up ----
  if (tid == 0) {
    for (int s = 0; s < kMaxStages; ++s) {
      mbar_init(smem_u32(&hdr->full[s]), kP16ProducerThreads + 1);   // cp.async arrivals + the TMA thread's expect_tx
      mbar_init(smem_u32(&hdr->empty[s]), 1);
    }
    mbar_init(smem_u32(&hdr->acc1_full), 1);
    mbar_init(smem_u32(&hdr->y_ready), kP16ConvertWarps);
    mbar_init(smem_u32(&hdr->s_done), 1);
    for (int b = 0; b < 4; ++b) mbar_init(smem_u32(&hdr->acc2_full[b]), 1);
    for (int b = 0; b < 2; ++b) mbar_init(smem_u32(&hdr->acc2_empty[b]), kP16ScatterWarps / 2);
    mbar_init(smem_u32(&hdr->drain), 1);
    fence_mbar_init();
    hdr->abort_flag = (p.status && (*reinterpret_cast<volatile int32_t*>(p.status) & EGS_STATUS_PIPELINE_TIMEOUT)) ? 1u : 0u;
    if (smem_misaligned(smem_raw)) {
      hdr->abort_flag = 1u;
      if (p.status) atomicOr(p.status, EGS_STATUS_INTERNAL);
    }
  }
  if (warp == kP16WarpG) {
    tmem_alloc(smem_u32(&hdr->tmem_base), kP16TmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = hdr->tmem_base;
  const bool run = (hdr->abort_flag == 0u);

  if (!run) {
    // fall through to the common exit
  } else if (warp < kP16ProducerWarps) {
    // =========================== producers ===========================
    // The dense weight tiles come by TMA (one thread, a few box loads per stage, written in the 128-byte swizzle the
    // tensor core reads); the 256 producer threads only gather the Src rows of the G stages with 16-byte cp.async.
    // full[slot] therefore collects 256 cp.async arrivals plus one expect_tx arrival and the TMA byte count.
    //   W1, CN layout [E, C1, N1]: map dims {N1, C1, E}, box {64 n, 64 c}: one box per 64-wide segment column
    //   W1, NC layout [E, N1, C1]: map dims {C1, N1, E}, box {64 c, N1 n}: one box
    //   W2, CN layout [E, N1, N2]: map dims {N2, N1, E}, box {64 n, N1 j}: one box
    //   W2, NC layout [E, N2, N1]: map dims {N1, N2, E}, box {64 j, 64 n}: one box per 64-element contraction segment
    const char* Src = static_cast<const char*>(p.Src);
    const long long rb_src = static_cast<long long>(p.C1) * ES;
    const int cc = tid & 7, r0 = tid >> 3;
    const uint32_t rc_dst0 = static_cast<uint32_t>(r0) * 128u + (static_cast<uint32_t>(cc ^ (r0 & 7)) << 4);
    bool alive = true;
    P16Ring ring;
    const char* a_src[kTileM / 32];              // gather sources of the row block whose G stages are being issued
    uint32_t a_mask = 0;
    auto look_up = [&](const P16Block& blk) {
      a_mask = 0;
#pragma unroll
      for (int i = 0; i < kTileM / 32; ++i) {
        int tok, slot;
        p16_rows(p, blk.e, blk.m0 + r0 + 32 * i, tok, slot, false);
        a_src[i] = Src + (tok >= 0 ? static_cast<long long>(tok) * rb_src : 0ll) + cc * 16;
        if (tok >= 0) a_mask |= 1u << i;
      }
    };
    auto acquire = [&]() -> uint32_t {           // waits for the next ring slot; returns its address (0 = aborting)
      if (ring.round > 0)
        alive = mbar_wait_warp(smem_u32(&hdr->empty[ring.slot]), (ring.round - 1) & 1, abort_flag, p.status, lane);
      return alive ? ring0 + static_cast<uint32_t>(ring.slot) * slot_bytes : 0u;
    };
    auto publish = [&]() {
      cp_async_mbar_arrive_noinc(smem_u32(&hdr->full[ring.slot]));
      ring.advance(stages);
    };
    // G stage ks of row block blk: [A: 128 gathered rows x 128 bytes | B: W1 tile]
    auto produce_g = [&](const P16Block& blk, int ks) {
      const uint32_t base = acquire();
      if (!alive) return;
      if (tid == 0) {
        const uint32_t bar = smem_u32(&hdr->full[ring.slot]);
        const uint32_t bbase = base + a_bytes;
        if (w_nc) {
          mbar_arrive_expect_tx(bar, static_cast<uint32_t>(p.N1) * 128u);
          tma_load_3d(bbase, &map_w1, ks * KE, 0, blk.e, bar);
        } else {
          mbar_arrive_expect_tx(bar, static_cast<uint32_t>(nseg_b1) * (KE * 128u));
          for (int j = 0; j < nseg_b1; ++j) tma_load_3d(bbase + static_cast<uint32_t>(j) * (KE * 128u), &map_w1, j * 64, ks * KE, blk.e, bar);
        }
      }
      const long long koff = static_cast<long long>(ks) * 128;
      if ((ks + 1) * KE <= p.C1 && a_mask == 0xFu) {
#pragma unroll
        for (int i = 0; i < kTileM / 32; ++i) cp_async16_full(base + rc_dst0 + i * 4096u, a_src[i] + koff);
      } else {
        const bool kvalid = koff + cc * 16 < rb_src;
#pragma unroll
        for (int i = 0; i < kTileM / 32; ++i) {
          const bool v = kvalid && ((a_mask >> i) & 1u);
          cp_async16(base + rc_dst0 + i * 4096u, v ? a_src[i] + koff : Src, v ? 16u : 0u);
        }
      }
      publish();
    };
    // S stage nt of row block blk: the W2 tile of output columns [nt*64, +64), whole contraction
    auto produce_s = [&](const P16Block& blk, int nt) {
      const uint32_t base = acquire();
      if (!alive) return;
      if (tid == 0) {
        const uint32_t bar = smem_u32(&hdr->full[ring.slot]);
        const int n0 = nt * kP16NT;
        if (w_nc) {
          mbar_arrive_expect_tx(bar, static_cast<uint32_t>(nseg_b2) * (kP16NT * 128u));
          for (int j = 0; j < nseg_b2; ++j) tma_load_3d(base + static_cast<uint32_t>(j) * (kP16NT * 128u), &map_w2, j * 64, n0, blk.e, bar);
        } else {
          mbar_arrive_expect_tx(bar, static_cast<uint32_t>(p.N1) * 128u);
          tma_load_3d(base, &map_w2, n0, 0, blk.e, bar);
        }
      }
      publish();
    };
    if (static_cast<int>(blockIdx.x) < row_blocks) {
      const P16Block first = p16_block(p, blockIdx.x, m_tiles);
      look_up(first);
      for (int ks = 0; ks < nk1 && alive; ++ks) produce_g(first, ks);
    }
    for (int rb = blockIdx.x; rb < row_blocks && alive; rb += gridDim.x) {
      const P16Block blk = p16_block(p, rb, m_tiles);
      const bool has_next = rb + static_cast<int>(gridDim.x) < row_blocks;
      P16Block nxt = blk;
      if (has_next) {
        nxt = p16_block(p, rb + gridDim.x, m_tiles);
        look_up(nxt);
      }
      for (int i = 0; i < steps && alive; ++i) {
        if (i < n2) produce_s(blk, i);
        if (has_next && i < nk1 && alive) produce_g(nxt, i);
      }
    }
    cp_async_wait_all();
  } else if (warp < kP16ProducerWarps + kP16ConvertWarps) {
    // =========================== converters: acc1 -> Y ===========================
    const int q = warp & 3;                              // TMEM lane group of this warp
    const uint32_t lane_base = static_cast<uint32_t>(q * 32) << 16;
    T* mid = static_cast<T*>(p.Mid);
    bool alive = true;
    int tcnt = 0;
    for (int rb = blockIdx.x; rb < row_blocks && alive; rb += gridDim.x, ++tcnt) {
      const P16Block blk = p16_block(p, rb, m_tiles);
      int tok, slot;
      p16_rows(p, blk.e, blk.m0 + q * 32 + lane, tok, slot, true);
      // acc1 of this row block is complete, and the S tiles of the previous one no longer read Y
      alive = mbar_wait_warp(smem_u32(&hdr->acc1_full), tcnt & 1, abort_flag, p.status, lane);
      if (alive && tcnt > 0) alive = mbar_wait_warp(smem_u32(&hdr->s_done), (tcnt - 1) & 1, abort_flag, p.status, lane);
      if (!alive) break;
      tc_fence_after();
      T* dst = mid + static_cast<long long>(slot >= 0 ? slot : 0) * p.N1;
      for (int c = 0; c * 32 < p.N1; ++c) {
        uint32_t v[32];
        tmem_ld32(tmem_base + lane_base + kP16ColAcc1 + static_cast<uint32_t>(c * 32), v);
        tmem_ld_wait();
        uint32_t pk[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) pk[j] = pack2(mid, v[2 * j], v[2 * j + 1]);
        tmem_st16(tmem_base + lane_base + kP16ColY + static_cast<uint32_t>(c * 16), pk);
        if (slot >= 0) {
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (c * 32 + j * 8 < p.N1)
              *reinterpret_cast<uint4*>(dst + c * 32 + j * 8) = make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
        }
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&hdr->y_ready));
    }
  } else if (warp < kP16WarpG) {
    // =========================== scatter epilogue: acc2 -> token rows ===========================
    // Group g takes the tile pairs {4j + 2g, 4j + 2g + 1} of every row block: two adjacent 64-column tiles are staged
    // side by side and leave as ONE 256-byte bulk reduction per row (the copy engine's rate is per operation).  While
    // one group's operations queue up in the copy engine the other group reads and converts the next pair.
    const int q = warp & 3;
    const int sw = warp - (kP16ProducerWarps + kP16ConvertWarps);
    const int grp = sw >> 2;
    const uint32_t lane_base = static_cast<uint32_t>(q * 32) << 16;
    const uint32_t my_area = staging0 + static_cast<uint32_t>(sw) * kP16BufBytes;
    const uint32_t srow = my_area + static_cast<uint32_t>(lane) * kP16RowPitch;
    T* out16 = static_cast<T*>(p.Out16);
    const bool direct16 = p.plan != nullptr && *p.plan == 0;
    bool alive = true;
    uint32_t seen = 0;                                   // bit b: parity of the tiles this group has taken from acc2[b]
    for (int rb = blockIdx.x; rb < row_blocks && alive; rb += gridDim.x) {
      const P16Block blk = p16_block(p, rb, m_tiles);
      int tok, slot;
      p16_rows(p, blk.e, blk.m0 + q * 32 + lane, tok, slot, false);
      for (int nt = 0; nt < n2 && alive; ++nt) {
        if (((nt >> 1) & 1) != grp) continue;
        const int buf = nt & 1;                          // tile nt of every row block goes through acc2[nt & 1]
        const int n0 = nt * kP16NT;
        const int bn = min(kP16NT, ((p.N2 - n0) + 15) & ~15);
        // a barrier of its own per (group, buffer): this group sees every one of its completions, in order
        alive = mbar_wait_warp(smem_u32(&hdr->acc2_full[2 * grp + buf]), (seen >> buf) & 1u, abort_flag, p.status, lane);
        seen ^= 1u << buf;
        if (!alive) break;
        tc_fence_after();
        const uint32_t acc = tmem_base + lane_base + kP16ColAcc2 + static_cast<uint32_t>(buf * kP16NT);
        if (direct16) {
          const int half = nt & 1;                       // position of this tile in its pair
          if (half == 0) bulk_wait_read_0();             // this warp's previous reduction has been read out of the buffer
          uint32_t v0[32], v1[32];
          tmem_ld32(acc, v0);
          if (bn > 32) tmem_ld32(acc + 32u, v1);
          tmem_ld_wait();
          // the accumulator has been read: hand it back before anything else
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&hdr->acc2_empty[buf]));
          const uint32_t dst = srow + static_cast<uint32_t>(half) * 128u;
#pragma unroll
          for (int j = 0; j < 4; ++j)
            asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(dst + j * 16u),
                         "r"(pack2(out16, v0[8 * j], v0[8 * j + 1])), "r"(pack2(out16, v0[8 * j + 2], v0[8 * j + 3])),
                         "r"(pack2(out16, v0[8 * j + 4], v0[8 * j + 5])), "r"(pack2(out16, v0[8 * j + 6], v0[8 * j + 7]))
                         : "memory");
          if (bn > 32) {
#pragma unroll
            for (int j = 0; j < 4; ++j)
              asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(dst + 64u + j * 16u),
                           "r"(pack2(out16, v1[8 * j], v1[8 * j + 1])), "r"(pack2(out16, v1[8 * j + 2], v1[8 * j + 3])),
                           "r"(pack2(out16, v1[8 * j + 4], v1[8 * j + 5])), "r"(pack2(out16, v1[8 * j + 6], v1[8 * j + 7]))
                           : "memory");
          }
          if (half == 1 || nt == n2 - 1) {
            fence_proxy_async_smem();
            const int g0 = (nt - half) * kP16NT;         // first column of the pair
            const int ncols = min((half + 1) * kP16NT, p.N2 - g0);
            if (tok >= 0 && ncols > 0)
              bulk_reduce_add(out16 + static_cast<long long>(tok) * p.N2 + g0, srow, static_cast<uint32_t>(ncols) * 2u);
            bulk_commit();
          }
        } else {
          for (int c = 0; c * 32 < bn; ++c) {
            const int col0 = n0 + c * 32;
            warp_block_emit(acc + static_cast<uint32_t>(c * 32), my_area, lane, true,
                            [&](int row, int cj, uint32_t x0, uint32_t x1, uint32_t x2, uint32_t x3) {
                              const int ro = __shfl_sync(0xffffffffu, tok, row);
                              const int col = col0 + cj;
                              if (ro >= 0 && col < p.N2) red4(p.Dst + static_cast<long long>(ro) * p.N2 + col, x0, x1, x2, x3);
                            });
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&hdr->acc2_empty[buf]));
        }
      }
    }
    if (direct16) bulk_wait_all();                       // shared memory must outlive the copy engine's reads
  } else if (warp == kP16WarpG) {
    // =========================== MMA issuer of the G stages ===========================
    if (lane == 0) {
      constexpr uint32_t fmt = Elem<T>::fmt;
      const uint32_t idesc1 = make_idesc(fmt, 0u, w_nc ? 0u : 1u, kTileM, static_cast<uint32_t>(p.BN1));
      const uint32_t acc1 = tmem_base + kP16ColAcc1;
      // descriptors without a start address; the ring slot's address (16-byte units) is added per stage
      const uint64_t a_desc0 = make_smem_desc(0u, 16u, 1024u);
      const uint64_t b1_desc0 = w_nc ? make_smem_desc(0u, 16u, 1024u) : make_smem_desc(0u, KE * 128u, 1024u);
      const uint32_t a_adv = 32u >> 4, b1_adv = (w_nc ? 32u : UK * 128u) >> 4;
      const int nk1_full = p.C1 / KE;             // stages with all four contraction steps
      bool ok = true;
      P16Ring ring;
      int tcnt = 0;
      auto mma_g = [&](int ks) {                 // one G stage into acc1
        ok = mbar_wait(smem_u32(&hdr->full[ring.slot]), ring.round & 1, abort_flag, p.status);
        if (!ok) return;
        const uint32_t base = ring0 + static_cast<uint32_t>(ring.slot) * slot_bytes;
        const uint64_t ad = a_desc0 + (base >> 4);
        const uint64_t bd = b1_desc0 + ((base + a_bytes) >> 4);
        if (ks < nk1_full) {
          umma_ss_f16_x4(acc1, ad, bd, a_adv, b1_adv, idesc1, ks > 0 ? 1u : 0u);
        } else {
          const int nkq = (p.C1 - ks * KE + UK - 1) / UK;
          for (int kq = 0; kq < nkq; ++kq)
            umma<false>(acc1, ad + static_cast<uint64_t>(kq) * a_adv, bd + static_cast<uint64_t>(kq) * b1_adv, idesc1,
                        (ks > 0 || kq > 0) ? 1u : 0u);
        }
        umma_commit(smem_u32(&hdr->empty[ring.slot]));
        ring.advance(stages);
      };
      // A stage of the other issuing lane: this lane still waits for it to land before it moves on.  A parity wait can
      // only tell the current phase of a barrier from the one before, so a lane that skipped phases of full[slot] could
      // mistake an older completion for its own stage's.
      auto pass_foreign = [&]() {
        ok = mbar_wait(smem_u32(&hdr->full[ring.slot]), ring.round & 1, abort_flag, p.status);
        ring.advance(stages);
      };
      if (static_cast<int>(blockIdx.x) < row_blocks) {
        for (int ks = 0; ks < nk1 && ok; ++ks) mma_g(ks);
        if (ok) umma_commit(smem_u32(&hdr->acc1_full));
      }
      for (int rb = blockIdx.x; rb < row_blocks && ok; rb += gridDim.x, ++tcnt) {
        const bool has_next = rb + static_cast<int>(gridDim.x) < row_blocks;
        if (has_next) {
          // acc1 has been read (Y(t) is complete) before G(t+1) overwrites it
          ok = mbar_wait(smem_u32(&hdr->y_ready), tcnt & 1, abort_flag, p.status);
          if (!ok) break;
          tc_fence_after();
        }
        for (int i = 0; i < steps && ok; ++i) {
          if (i < n2) pass_foreign();                    // the S lane's stage
          if (has_next && i < nk1 && ok) mma_g(i);
        }
        if (has_next && ok) umma_commit(smem_u32(&hdr->acc1_full));
      }
    }
    __syncwarp();
  } else {
    // =========================== MMA issuer of the S tiles ===========================
    if (lane == 0) {
      constexpr uint32_t fmt = Elem<T>::fmt;
      const uint32_t ytm = tmem_base + kP16ColY;
      const uint64_t b2_desc0 = w_nc ? make_smem_desc(0u, 16u, 1024u) : make_smem_desc(0u, kP16NT * 128u, 1024u);
      const uint32_t b2_adv = (w_nc ? 32u : UK * 128u) >> 4;
      const uint32_t b2_jump = w_nc ? ((kP16NT * 128u) >> 4) - 4u * b2_adv : 0u;   // K-major: the 5th step starts the next segment
      const uint32_t b2_group = w_nc ? 2u * ((kP16NT * 128u) >> 4) : 8u * b2_adv;  // eight steps further on
      const int nkq2 = p.N1 / UK;                // contraction steps per S tile (at most 16)
      bool ok = true;
      P16Ring ring;
      int tcnt = 0;
      uint32_t used = 0, par_e = 0;              // per accumulator: used before; parity of the release to wait for next
      // (see the G lane: stages of the other lane are waited for too, so that no phase of full[slot] is skipped)
      auto pass_foreign = [&]() {
        ok = mbar_wait(smem_u32(&hdr->full[ring.slot]), ring.round & 1, abort_flag, p.status);
        ring.advance(stages);
      };
      for (int ks = 0; ks < nk1 && ok; ++ks) pass_foreign();           // the G stages of the first row block
      for (int rb = blockIdx.x; rb < row_blocks && ok; rb += gridDim.x, ++tcnt) {
        const bool has_next = rb + static_cast<int>(gridDim.x) < row_blocks;
        ok = mbar_wait(smem_u32(&hdr->y_ready), tcnt & 1, abort_flag, p.status);
        if (!ok) break;
        tc_fence_after();
        for (int i = 0; i < steps && ok; ++i) {
          if (i < n2) {
            const int buf = i & 1, gb = 2 * ((i >> 1) & 1) + buf;
            if ((used >> buf) & 1u) {                      // the previous tile in this accumulator has been read
              ok = mbar_wait(smem_u32(&hdr->acc2_empty[buf]), (par_e >> buf) & 1u, abort_flag, p.status);
              if (!ok) break;
              par_e ^= 1u << buf;
              tc_fence_after();
            }
            used |= 1u << buf;
            ok = mbar_wait(smem_u32(&hdr->full[ring.slot]), ring.round & 1, abort_flag, p.status);
            if (!ok) break;
            const uint32_t base = ring0 + static_cast<uint32_t>(ring.slot) * slot_bytes;
            const int bn = min(kP16NT, ((p.N2 - i * kP16NT) + 15) & ~15);
            const uint32_t idesc2 = make_idesc(fmt, 0u, w_nc ? 0u : 1u, kTileM, static_cast<uint32_t>(bn));
            const uint32_t d = tmem_base + kP16ColAcc2 + static_cast<uint32_t>(buf * kP16NT);
            const uint64_t bd = b2_desc0 + (base >> 4);
            if (nkq2 == 16) {
              umma_ts_f16_x8(d, ytm, bd, b2_adv, b2_jump, idesc2, 0u);
              umma_ts_f16_x8(d, ytm + 64u, bd + b2_group, b2_adv, b2_jump, idesc2, 1u);
            } else {
              for (int kq = 0; kq < nkq2; ++kq)
                umma_ts_f16(d, ytm + static_cast<uint32_t>(kq * 8),
                            bd + static_cast<uint64_t>(kq) * b2_adv + static_cast<uint64_t>(kq >> 2) * b2_jump, idesc2, kq > 0 ? 1u : 0u);
            }
            umma_commit(smem_u32(&hdr->empty[ring.slot]));
            umma_commit(smem_u32(&hdr->acc2_full[gb]));
            ring.advance(stages);
          }
          if (has_next && i < nk1 && ok) pass_foreign();   // the G lane's stage
        }
        // completes when the S tiles of this row block no longer read Y
        if (ok) umma_commit(smem_u32(&hdr->s_done));
      }
    }
    __syncwarp();
  }

  // ---- common exit ----
  tc_fence_before();
  __syncthreads();
  if (warp == kP16WarpG) tmem_release(tmem_base, kP16TmemCols, smem_u32(&hdr->drain), abort_flag, lane);
}

constexpr size_t kP16SmemMax = 227 * 1024;
constexpr int kP16SmCount = 148;

}  // namespace

// Fills BN1 / slot_bytes / stages and returns the dynamic shared memory size; 0 = shape not taken.
size_t configure_tensor_pair16(FusedParams& p) {
  if (p.C1 < 8 || p.C1 % 8 != 0 || p.N2 < 8 || p.N2 % 8 != 0) return 0;     // 16-byte row pitches
  if (p.N1 < 16 || p.N1 > 256 || p.N1 % 16 != 0) return 0;                  // Y is whole tcgen05.mma contraction steps
  p.BN1 = p.N1;
  p.BN2 = kP16NT;
  const bool nc = (p.w_layout == EGS_W_NC);
  const size_t a_bytes = static_cast<size_t>(kTileM) * 128;
  const size_t nseg1 = (static_cast<size_t>(p.BN1) * 2 + 127) / 128;
  const size_t b1 = nc ? static_cast<size_t>(p.BN1) * 128 : nseg1 * 64 * 128;
  const size_t b2 = static_cast<size_t>((p.N1 + 63) / 64) * 64 * 128;      // S stage: contraction rows (or segments) x 128 bytes
  size_t slot = a_bytes + b1 > b2 ? a_bytes + b1 : b2;
  slot = (slot + 1023) & ~static_cast<size_t>(1023);
  size_t ns = (kP16SmemMax - kP16RingOffset) / slot;
  if (ns > static_cast<size_t>(kMaxStages)) ns = kMaxStages;
  if (ns < 2) return 0;
  p.slot_bytes = static_cast<uint32_t>(slot);
  p.stages = static_cast<int>(ns);
  return kP16RingOffset + ns * slot;
}

// The opt-in to large dynamic shared memory is per kernel function and device: done once per host thread and device.
template <typename T>
static cudaError_t p16_smem_optin() {
  static thread_local int done_device = -1;
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  if (done_device == dev) return cudaSuccess;
  err = cudaFuncSetAttribute(tensor_pair16_persistent_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(kP16SmemMax));
  if (err == cudaSuccess) done_device = dev;
  return err;
}

cudaError_t launch_tensor_pair16(const FusedParams& p, int dtype, size_t smem_bytes, cudaStream_t st) {
  // tensor maps of the two weight tensors (see the producers' comment for the geometry)
  const bool nc = (p.w_layout == EGS_W_NC);
  TensorMap3 m1, m2;
  const unsigned long long e = static_cast<unsigned long long>(p.E);
  const unsigned long long d1[3] = {static_cast<unsigned long long>(nc ? p.C1 : p.N1), static_cast<unsigned long long>(nc ? p.N1 : p.C1), e};
  const unsigned b1[3] = {64u, nc ? static_cast<unsigned>(p.N1) : 64u, 1u};
  const unsigned long long d2[3] = {static_cast<unsigned long long>(nc ? p.N1 : p.N2), static_cast<unsigned long long>(nc ? p.N2 : p.N1), e};
  const unsigned b2[3] = {64u, nc ? 64u : static_cast<unsigned>(p.N1), 1u};
  if (!encode_tensor_map_16bit(&m1, p.W1, d1, b1) || !encode_tensor_map_16bit(&m2, p.W2, d2, b2)) return cudaErrorInvalidValue;
  const int row_blocks = p.E * ((p.M + kTileM - 1) / kTileM);
  dim3 grid(row_blocks < kP16SmCount ? row_blocks : kP16SmCount);
  dim3 block(kP16Threads);
  cudaError_t err;
  if (dtype == EGS_F16) {
    err = p16_smem_optin<__half>();
    if (err == cudaSuccess) tensor_pair16_persistent_kernel<__half><<<grid, block, smem_bytes, st>>>(p, m1, m2);
  } else {
    err = p16_smem_optin<__nv_bfloat16>();
    if (err == cudaSuccess) tensor_pair16_persistent_kernel<__nv_bfloat16><<<grid, block, smem_bytes, st>>>(p, m1, m2);
  }
  if (err != cudaSuccess) return err;
  count_launch();
  return cudaGetLastError();
}

}  // namespace egs
