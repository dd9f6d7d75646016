// Operator G for 16-bit tensors on PAIRS of SMs (sm_100a): thread-block clusters of two CTAs and tcgen05.mma.cta_group::2.
//
// Selected only on request (EGS_PATH_PAIRED): at the benchmark's shapes it measured 164-170 us against 152-158 us of the
// single-CTA kernel it was written to replace.
// The idea: a 256-row CTA of the single-CTA kernel stages the whole W[e] (C x N) for its 256 gathered rows, and tensor memory
// (512 columns) allows no taller CTA.  Here two CTAs of one cluster work on 512 expert rows of one expert together: each
// gathers its own 256 rows (A operand, two 128-row tiles) but stages only HALF of every W tile (N/2 columns); the pair's MMA
// instructions (M = 256: 128 rows from each CTA) read the B operand from both halves.  W bytes per expert row halve, A bytes
// stay: -25 % staged bytes, -30 % shared-memory traffic per flop, and the W halves come through the TMA unit, which leaves
// the load/store unit to the gathers.  What it loses again: the TMA unit needs about 9 clocks per 128-byte row of a box, the
// peer's "stage landed" events and the leader's commits cross the pair, and the read-out's row-per-thread stores compete
// with the gathers for the load/store unit.
//
// Persistent: 74 CTA pairs (one CTA per SM) walk the list of (expert, 512-row block) tiles; the shared-memory ring runs on
// across tiles.
//   warps 0..3   producers: 16-byte cp.async gathers of the CTA's 256 token rows (row indices fetched one tile ahead); thread 0
//                also issues the TMA box loads of this CTA's half of the W tile
//   warp  4      TMEM allocation (cta_group::2: the same warp of both CTAs); in the leader CTA (cluster rank 0) one lane issues
//                every tcgen05.mma of the pair and commits to the barriers of both CTAs; in the peer CTA (rank 1) one lane
//                is the relay: it waits for each stage of the peer to land and arrives on the leader's `peer_full[s]`
//                barrier (cp.async can only signal a barrier of its own CTA)
//   warp  21     index warp: looks up the token rows of the next tiles (Ind) and leaves them in shared memory for the producers
//   warps 5..20  epilogue: each warp reads its 32 rows x 128 columns of one accumulator into registers (packed to 16 bits),
//                releases the accumulator at once - with N = 256 tensor memory holds one buffer of the two accumulators, so
//                the pair's next MMAs wait for exactly this read-out - and only then writes its rows (+ bias) with 32-byte
//                stores (a thread owns a row: that is how tensor memory hands it out)
// Barriers per CTA: full[s] (own data landed), empty[s] (the pair's MMAs on stage s are complete: committed by the leader to
// both CTAs), peer_full[s] (leader only), acc_full[b] (a tile's MMAs are complete, committed to both CTAs), acc_empty[b]
// (leader only: the 32 epilogue warps of the pair have read buffer b).  No load in this file is shared between CTAs or
// multi-destination: every CTA fetches its own operand bytes.  Every wait is bounded; when one runs out the CTA raises its
// abort flag and EGS_STATUS_PIPELINE_TIMEOUT, its roles fall through to the exit, and the partner's waits on it run out in turn.
#include "egs_tcgen05.cuh"

namespace egs {

namespace {

constexpr int kG2ProducerWarps = 4, kG2ProducerThreads = kG2ProducerWarps * 32;
constexpr int kG2MmaWarp = kG2ProducerWarps, kG2EpilogueWarp0 = kG2ProducerWarps + 1;
constexpr int kG2EpilogueWarps = 16;             // 4 TMEM lane groups x 2 accumulators x 2 column halves
constexpr int kG2IndexWarp = kG2EpilogueWarp0 + kG2EpilogueWarps;
constexpr int kG2Threads = (kG2IndexWarp + 1) * 32;
constexpr int kG2Rows = 2 * kTileM;              // expert rows per CTA (two accumulators)
constexpr int kG2RowsPerThread = kG2Rows * 8 / kG2ProducerThreads;    // 8 threads per 128-byte row piece
constexpr int kG2Pairs = 74;                     // CTA pairs of the persistent grid: one CTA per SM
constexpr uint32_t kG2HeaderBytes = 3072;
constexpr size_t kG2SmemMax = 227 * 1024;

struct __align__(16) G2Header {
  unsigned long long full[kMaxStages];
  unsigned long long empty[kMaxStages];
  unsigned long long peer_full[kMaxStages];
  unsigned long long acc_full[2];  // per accumulator buffer: the pair's MMAs of a tile are complete (committed to both CTAs)
  unsigned long long acc_empty[2]; // leader's copy: the epilogue warps of both CTAs have read the buffer
  unsigned long long rows_full[2];   // the index warp has filled rows[b] for a tile
  unsigned long long rows_empty[2];  // the producer threads have taken their rows out of rows[b]
  unsigned long long drain;
  uint32_t tmem_base;
  uint32_t abort_flag;
  int rows[2][kG2Rows];              // token row (b*T + t) of each of the CTA's tile rows, -1 = masked; two tiles deep
};
static_assert(sizeof(G2Header) <= kG2HeaderBytes, "header does not fit");

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `local_addr` (an address in this CTA's shared memory) in the CTA of rank `rank`
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// one 32-byte store (a whole sector); the address must be 32-byte aligned
__device__ __forceinline__ void store_32bytes(void* dst, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t a4, uint32_t a5,
                                              uint32_t a6, uint32_t a7) {
  asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(dst), "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(a4), "r"(a5),
               "r"(a6), "r"(a7)
               : "memory");
}
// commit of the pair's MMAs issued so far to ONE barrier, which may live in either CTA (shared::cluster address)
__device__ __forceinline__ void umma2_commit(uint32_t cluster_bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar) : "memory");
}
// four contraction steps of the pair's MMA (M = 256: 128 rows of each CTA; B = N/2 columns from each CTA)
__device__ __forceinline__ void umma2_ss_f16_x4(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t a_adv, uint32_t b_adv,
                                                uint32_t idesc, uint32_t accumulate_first) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t.reg .b64 aa, bb, a, b;\n\t"
      "setp.ne.b32 p, %6, 0;\n\tsetp.eq.b32 q, 0, 0;\n\t"
      "cvt.u64.u32 aa, %3;\n\tcvt.u64.u32 bb, %4;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %5, p;\n\t"
      "add.u64 a, %1, aa;\n\tadd.u64 b, %2, bb;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], a, b, %5, q;\n\t"
      "add.u64 a, a, aa;\n\tadd.u64 b, b, bb;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], a, b, %5, q;\n\t"
      "add.u64 a, a, aa;\n\tadd.u64 b, b, bb;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], a, b, %5, q;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(a_adv), "r"(b_adv), "r"(idesc), "r"(accumulate_first)
      : "memory");
}
__device__ __forceinline__ void umma2_ss_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// The tile list of one CTA pair: tiles pair, pair + npairs, ... of E x nrb tiles (512 expert rows of one expert each).
struct G2Tiles {
  int ntiles, nrb, E, expert_fastest;
  __device__ __forceinline__ void locate(int t, int& e, int& rb) const {
    if (expert_fastest) { rb = t / E; e = t - rb * E; }      // experts fastest: the token rows of a batch block stay hot in L2
    else { e = t / nrb; rb = t - e * nrb; }                  // row blocks fastest: W[e] stays hot
  }
};

template <typename T>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kG2Threads, 1) tensor_gather2_kernel(RowGemmParams p, const __grid_constant__ TensorMap3 map_w) {
  constexpr int ES = 2, KE = 64, UK = 16;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  G2Header* hdr = reinterpret_cast<G2Header*>(smem_raw);
  const uint32_t smem0 = smem_u32(smem_raw);
  const uint32_t ring0 = smem0 + kG2HeaderBytes;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = (rank == 0);
  const bool w_nc = (p.w_layout == EGS_W_NC);
  const int nh = p.BN / 2;                                   // columns of W this CTA stages
  const int nseg_h = (nh * ES + 127) / 128;                  // 128-byte segment columns of the half tile in CN layout
  const uint32_t a_bytes = kG2Rows * 128u;
  const uint32_t b_bytes = w_nc ? static_cast<uint32_t>(nh) * 128u : static_cast<uint32_t>(nseg_h) * (KE * 128u);
  const uint32_t stage_bytes = (a_bytes + b_bytes + 1023u) & ~1023u;
  const int stages = p.stages;
  const int nk = (p.C + KE - 1) / KE;
  const uint32_t acc_cols = tmem_cols_for(p.BN);
  // two buffers of the two accumulators when tensor memory (512 columns) holds them
  const uint32_t nbuf = (4u * acc_cols <= 512u) ? 2u : 1u;
  const uint32_t tmem_cols = nbuf * 2u * acc_cols;
  volatile uint32_t* abort_flag = &hdr->abort_flag;
  G2Tiles tiles;
  tiles.nrb = (p.M + 2 * kG2Rows - 1) / (2 * kG2Rows);
  tiles.E = p.E;
  tiles.ntiles = tiles.nrb * p.E;
  tiles.expert_fastest = p.expert_fastest;
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;

  // ---- set-up ----
  if (tid == 0) {
    for (int s = 0; s < kMaxStages; ++s) {
      mbar_init(smem_u32(&hdr->full[s]), kG2ProducerThreads + 1);   // cp.async arrivals + the TMA thread's expect_tx
      mbar_init(smem_u32(&hdr->empty[s]), 1);
      mbar_init(smem_u32(&hdr->peer_full[s]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&hdr->acc_full[i]), 1);
      mbar_init(smem_u32(&hdr->acc_empty[i]), 2 * kG2EpilogueWarps);     // the epilogue warps of both CTAs (leader's copy is used)
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&hdr->rows_full[i]), 1);
      mbar_init(smem_u32(&hdr->rows_empty[i]), kG2ProducerThreads);
    }
    mbar_init(smem_u32(&hdr->drain), 1);
    fence_mbar_init();
    hdr->abort_flag = (p.status && (*reinterpret_cast<volatile int32_t*>(p.status) & EGS_STATUS_PIPELINE_TIMEOUT)) ? 1u : 0u;
    if (smem_misaligned(smem_raw)) {
      hdr->abort_flag = 1u;
      if (p.status) atomicOr(p.status, EGS_STATUS_INTERNAL);
    }
  }
  __syncthreads();
  if (warp == kG2MmaWarp) {
    tmem_alloc2(smem_u32(&hdr->tmem_base), tmem_cols);
    tmem_relinquish2();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                    // both CTAs' barriers are initialised before anything crosses the pair
  tc_fence_after();
  const uint32_t tmem_base = hdr->tmem_base;
  const bool run = (hdr->abort_flag == 0u);

  if (!run) {
    // fall through to the common exit
  } else if (warp < kG2ProducerWarps) {
    // =========================== producers ===========================
    const char* A = static_cast<const char*>(p.A);
    const long long row_bytes_a = static_cast<long long>(p.C) * ES;
    const int cc = tid & 7, r0 = tid >> 3;                 // 16-byte chunk of the 128-byte piece; rows r0, r0 + 16, ...
    const uint32_t rc_dst0 = static_cast<uint32_t>(r0) * 128u + (static_cast<uint32_t>(cc ^ (r0 & 7)) << 4);
    constexpr uint32_t kRowStep = (kG2ProducerThreads / 8) * 128u;   // bytes between this thread's rows in the tile (16 rows)
    int tok[kG2RowsPerThread];
    bool alive = true;
    int slot = 0;
    uint32_t round = 0, tcnt = 0;
    for (int t = pair; t < tiles.ntiles && alive; t += npairs, ++tcnt) {
      int e, rb;
      tiles.locate(t, e, rb);
      // this thread's token rows, looked up by the index warp while the previous tile was loading
      const uint32_t rbuf = tcnt & 1u;
      alive = mbar_wait_warp(smem_u32(&hdr->rows_full[rbuf]), (tcnt >> 1) & 1, abort_flag, p.status, lane);
      if (!alive) break;
      bool all_rows = true;
#pragma unroll
      for (int i = 0; i < kG2RowsPerThread; ++i) {
        tok[i] = hdr->rows[rbuf][r0 + (kG2ProducerThreads / 8) * i];
        all_rows = all_rows && tok[i] >= 0;
      }
      mbar_arrive(smem_u32(&hdr->rows_empty[rbuf]));
      const char* a0 = A + cc * 16;
      for (int kt = 0; kt < nk && alive; ++kt) {
        if (round > 0) alive = mbar_wait_warp(smem_u32(&hdr->empty[slot]), (round - 1) & 1, abort_flag, p.status, lane);
        if (!alive) break;
        const uint32_t base = ring0 + static_cast<uint32_t>(slot) * stage_bytes;
        const uint32_t bar = smem_u32(&hdr->full[slot]);
        if (tid == 0) {
          const uint32_t bbase = base + a_bytes;
          mbar_arrive_expect_tx(bar, b_bytes);
          if (w_nc) {      // map dims {C, N, E}, box {64 c, N/2 rows}
            tma_load_3d(bbase, &map_w, kt * KE, static_cast<int>(rank) * nh, e, bar);
          } else {         // map dims {N, C, E}, box {64 n, 64 c}: one box per 64-wide segment column of this CTA's half
            for (int j = 0; j < nseg_h; ++j)
              tma_load_3d(bbase + static_cast<uint32_t>(j) * (KE * 128u), &map_w, static_cast<int>(rank) * nh + j * 64, kt * KE, e, bar);
          }
        }
        const char* ak = a0 + static_cast<long long>(kt) * 128;
        if ((kt + 1) * KE <= p.C && all_rows) {
#pragma unroll
          for (int i = 0; i < kG2RowsPerThread; ++i)
            cp_async16_full(base + rc_dst0 + i * kRowStep, ak + static_cast<long long>(tok[i]) * row_bytes_a);
        } else {
          const bool kvalid = static_cast<long long>(kt) * 128 + cc * 16 < row_bytes_a;
#pragma unroll
          for (int i = 0; i < kG2RowsPerThread; ++i) {
            const bool v = kvalid && tok[i] >= 0;
            cp_async16(base + rc_dst0 + i * kRowStep, v ? ak + static_cast<long long>(tok[i]) * row_bytes_a : A, v ? 16u : 0u);
          }
        }
        cp_async_mbar_arrive_noinc(bar);
        if (++slot == stages) {
          slot = 0;
          ++round;
        }
      }
    }
    cp_async_wait_all();
  } else if (warp == kG2MmaWarp) {
    // =========================== MMA issuer (leader CTA only) ===========================
    // (the same warp of the peer CTA relays the peer's "stage landed" events to the leader instead)
    if (leader && lane == 0) {
      constexpr uint32_t fmt = Elem<T>::fmt;
      // M = 256 (128 rows from each CTA), N = BN (half of the columns from each CTA's shared memory)
      const uint32_t idesc = make_idesc(fmt, 0u, w_nc ? 0u : 1u, 2 * kTileM, static_cast<uint32_t>(p.BN));
      const uint64_t a_desc0 = make_smem_desc(0u, 16u, 1024u);
      const uint64_t b_desc0 = w_nc ? make_smem_desc(0u, 16u, 1024u) : make_smem_desc(0u, KE * 128u, 1024u);
      const uint32_t a_adv = 32u >> 4, b_adv = (w_nc ? 32u : UK * 128u) >> 4;
      const uint32_t peer_empty0 = map_to_cta(smem_u32(&hdr->empty[0]), 1u);
      const uint32_t peer_acc_full0 = map_to_cta(smem_u32(&hdr->acc_full[0]), 1u);
      const int nk_full = p.C / KE;
      bool ok = true;
      int slot = 0;
      uint32_t round = 0, tcnt = 0;
      for (int t = pair; t < tiles.ntiles && ok; t += npairs, ++tcnt) {
        // the buffer has been read out in both CTAs by the epilogue warps of the tile that used it last
        const uint32_t buf = (nbuf == 2u) ? (tcnt & 1u) : 0u;
        const uint32_t use = (nbuf == 2u) ? (tcnt >> 1) : tcnt;          // how often the buffer has been used before
        if (use > 0) ok = mbar_wait(smem_u32(&hdr->acc_empty[buf]), (use - 1) & 1, abort_flag, p.status);
        if (!ok) break;
        tc_fence_after();
        for (int ks = 0; ks < nk && ok; ++ks) {
          ok = mbar_wait(smem_u32(&hdr->full[slot]), round & 1, abort_flag, p.status);
          if (ok) ok = mbar_wait(smem_u32(&hdr->peer_full[slot]), round & 1, abort_flag, p.status);
          if (!ok) break;
          tc_fence_after();
          const uint32_t base = (ring0 + static_cast<uint32_t>(slot) * stage_bytes) & 0x3FFFFu;   // offset inside the CTA
          const uint64_t bd = b_desc0 + ((base + a_bytes) >> 4);
#pragma unroll
          for (int mt = 0; mt < 2; ++mt) {
            const uint64_t ad = a_desc0 + ((base + static_cast<uint32_t>(mt) * (kTileM * 128u)) >> 4);
            const uint32_t d = tmem_base + (buf * 2u + static_cast<uint32_t>(mt)) * acc_cols;
            if (ks < nk_full) {
              umma2_ss_f16_x4(d, ad, bd, a_adv, b_adv, idesc, ks > 0 ? 1u : 0u);
            } else {
              const int nkq = (p.C - ks * KE + UK - 1) / UK;
              for (int kq = 0; kq < nkq; ++kq)
                umma2_ss_f16(d, ad + static_cast<uint64_t>(kq) * a_adv, bd + static_cast<uint64_t>(kq) * b_adv, idesc,
                             (ks > 0 || kq > 0) ? 1u : 0u);
            }
          }
          // the stage is free in BOTH CTAs once the pair's MMAs on it are complete
          umma2_commit(smem_u32(&hdr->empty[slot]));
          umma2_commit(peer_empty0 + static_cast<uint32_t>(slot) * 8u);
          if (++slot == stages) {
            slot = 0;
            ++round;
          }
        }
        if (ok) {
          umma2_commit(smem_u32(&hdr->acc_full[buf]));
          umma2_commit(peer_acc_full0 + buf * 8u);
        }
      }
    }
    // =========================== relay (peer CTA only): "my stage s has landed" -> leader ===========================
    if (!leader && lane == 0) {
      const uint32_t leader_peer_full0 = map_to_cta(smem_u32(&hdr->peer_full[0]), 0u);
      bool ok = true;
      int slot = 0;
      uint32_t round = 0;
      for (int t = pair; t < tiles.ntiles && ok; t += npairs) {
        for (int ks = 0; ks < nk && ok; ++ks) {
          ok = mbar_wait(smem_u32(&hdr->full[slot]), round & 1, abort_flag, p.status);
          if (!ok) break;
          fence_proxy_async_smem();
          mbar_arrive_cluster(leader_peer_full0 + static_cast<uint32_t>(slot) * 8u);
          if (++slot == stages) {
            slot = 0;
            ++round;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == kG2IndexWarp) {
    // =========================== index warp: token rows of the tiles, up to two tiles ahead ===========================
    bool alive = true;
    uint32_t tcnt = 0;
    for (int t = pair; t < tiles.ntiles && alive; t += npairs, ++tcnt) {
      const uint32_t rbuf = tcnt & 1u, use = tcnt >> 1;
      if (use > 0) alive = mbar_wait_warp(smem_u32(&hdr->rows_empty[rbuf]), (use - 1) & 1, abort_flag, p.status, lane);
      if (!alive) break;
      int e, rb;
      tiles.locate(t, e, rb);
      const int m0 = (rb * 2 + static_cast<int>(rank)) * kG2Rows;
      long long tk[kG2Rows / 32];
      int base_row[kG2Rows / 32];
#pragma unroll
      for (int i = 0; i < kG2Rows / 32; ++i) {       // all loads are issued before the first one is looked at
        const int m = m0 + lane + 32 * i;
        const bool on = m < p.M;
        const int b = on ? m / p.K : 0, k = on ? m - b * p.K : 0;
        base_row[i] = on ? b * p.T : -1;
        tk[i] = load_index(p.Ind, p.index_dtype, on ? static_cast<long long>(b * p.E + e) * p.K + k : 0ll);
      }
#pragma unroll
      for (int i = 0; i < kG2Rows / 32; ++i) {
        int row = -1;
        if (base_row[i] >= 0) {
          if (tk[i] >= 0 && tk[i] < p.T) row = base_row[i] + static_cast<int>(tk[i]);
          else if (p.status) atomicOr(p.status, EGS_STATUS_INDEX_OUT_OF_RANGE);
        }
        hdr->rows[rbuf][lane + 32 * i] = row;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&hdr->rows_full[rbuf]));
    }
  } else {
    // =========================== epilogue ===========================
    const int ew = warp - kG2EpilogueWarp0;
    const int lg = warp & 3;                            // TMEM lanes this warp may read: 32*lg .. 32*lg + 31
    const int mt = (ew >> 2) & 1, half = ew >> 3;       // which accumulator, which half of its 32-column blocks
    const uint32_t leader_acc_empty0 = map_to_cta(smem_u32(&hdr->acc_empty[0]), 0u);
    T* out = static_cast<T*>(p.Out);
    const int nblk = p.BN >> 5;                         // 32-column blocks of the tile (at most 8)
    const int c0 = half * ((nblk + 1) >> 1), c1 = half ? nblk : ((nblk + 1) >> 1);     // this warp's blocks [c0, c1): at most 4
    bool alive = true;
    uint32_t tcnt = 0;
    for (int t = pair; t < tiles.ntiles && alive; t += npairs, ++tcnt) {
      int e, rb;
      tiles.locate(t, e, rb);
      const int m = (rb * 2 + static_cast<int>(rank)) * kG2Rows + mt * kTileM + lg * 32 + lane;
      T* orow = nullptr;
      if (m < p.M) {
        const int b = m / p.K, k = m - b * p.K;
        orow = out + (static_cast<long long>(b * p.E + e) * p.K + k) * p.N;
      }
      const T* bias_row = p.bias ? static_cast<const T*>(p.bias) + static_cast<long long>(e) * p.N : nullptr;
      const uint32_t buf = (nbuf == 2u) ? (tcnt & 1u) : 0u;
      const uint32_t use = (nbuf == 2u) ? (tcnt >> 1) : tcnt;
      alive = mbar_wait_warp(smem_u32(&hdr->acc_full[buf]), use & 1, abort_flag, p.status, lane);
      if (!alive) break;
      tc_fence_after();
      const uint32_t trow = tmem_base + (static_cast<uint32_t>(lg * 32) << 16) + (buf * 2u + static_cast<uint32_t>(mt)) * acc_cols;
      // Three of the (at most four) blocks are held in registers, packed to 16 bits, and written after the release; the
      // register file has no room for the fourth, which is written straight away.
      uint32_t q[3][16];
      auto read_block = [&](int c, uint32_t (&dst)[16]) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t v[16];
          tmem_ld16(trow + static_cast<uint32_t>(c * 32 + h * 16), v);
          tmem_ld_wait();
          if (bias_row) {
#pragma unroll
            for (int i = 0; i < 16; i += 4) add_bias4<T>(bias_row + c * 32 + h * 16 + i, v[i], v[i + 1], v[i + 2], v[i + 3]);
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) dst[h * 8 + i] = pack2(out, v[2 * i], v[2 * i + 1]);
        }
      };
      auto write_block = [&](int c, const uint32_t (&src)[16]) {
        if (orow) {
          store_32bytes(orow + c * 32, src[0], src[1], src[2], src[3], src[4], src[5], src[6], src[7]);
          store_32bytes(orow + c * 32 + 16, src[8], src[9], src[10], src[11], src[12], src[13], src[14], src[15]);
        }
      };
#pragma unroll
      for (int j = 0; j < 3; ++j)
        if (c0 + j < c1) read_block(c0 + j, q[j]);
      if (c0 + 3 < c1) {
        const int c = c0 + 3;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t v[16];
          tmem_ld16(trow + static_cast<uint32_t>(c * 32 + h * 16), v);
          tmem_ld_wait();
          if (bias_row) {
#pragma unroll
            for (int i = 0; i < 16; i += 4) add_bias4<T>(bias_row + c * 32 + h * 16 + i, v[i], v[i + 1], v[i + 2], v[i + 3]);
          }
          if (orow)
            store_32bytes(orow + c * 32 + h * 16, pack2(out, v[0], v[1]), pack2(out, v[2], v[3]), pack2(out, v[4], v[5]), pack2(out, v[6], v[7]),
                          pack2(out, v[8], v[9]), pack2(out, v[10], v[11]), pack2(out, v[12], v[13]), pack2(out, v[14], v[15]));
        }
      }
      // this warp's reads of the accumulator are complete: tell the leader's MMA lane, then write the rows
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(leader_acc_empty0 + buf * 8u);
#pragma unroll
      for (int j = 0; j < 3; ++j)
        if (c0 + j < c1) write_block(c0 + j, q[j]);
    }
  }

  // ---- common exit: nobody leaves while the partner may still read its shared memory, write its tensor memory or
  // signal its barriers.  After an abort MMAs of the pair may still be in flight: the leader waits for them (bounded)
  // before the pair meets.
  tc_fence_before();
  __syncthreads();
  uint32_t safe = 1u;
  if (warp == kG2MmaWarp && *abort_flag) {
    if (lane == 0) {
      uint32_t ignore_abort = 0u;
      umma2_commit(smem_u32(&hdr->drain));
      safe = mbar_wait(smem_u32(&hdr->drain), 0u, &ignore_abort, nullptr) ? 1u : 0u;
    }
    safe = __shfl_sync(0xffffffffu, safe, 0);
  }
  cluster_sync_all();
  if (warp == kG2MmaWarp && safe) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, tmem_cols);
  }
}

}  // namespace

// Shapes this kernel takes: 16-bit tensors, N a multiple of 32 and at most 256 (one tile over N), C a multiple of 8,
// output rows 32-byte aligned (the epilogue's stores).  Fills BN / stages and returns the dynamic shared memory size;
// 0 = not taken.
size_t configure_tensor_gather2(RowGemmParams& p) {
  if (p.N < 32 || p.N > 256 || p.N % 32 != 0 || p.C < 8 || p.C % 8 != 0) return 0;
  if (reinterpret_cast<uintptr_t>(p.Out) % 32 != 0) return 0;
  p.BN = p.N;
  p.row_tiles = 2;
  const int nh = p.BN / 2;
  const size_t a_bytes = static_cast<size_t>(kG2Rows) * 128;
  const size_t nseg_h = (static_cast<size_t>(nh) * 2 + 127) / 128;
  const size_t b_bytes = (p.w_layout == EGS_W_NC) ? static_cast<size_t>(nh) * 128 : nseg_h * 64 * 128;
  const size_t stage = (a_bytes + b_bytes + 1023) & ~static_cast<size_t>(1023);
  const size_t fixed = kG2HeaderBytes;
  size_t ns = (kG2SmemMax - fixed) / stage;
  if (ns > static_cast<size_t>(kMaxStages)) ns = kMaxStages;
  if (ns < 2) return 0;
  p.stages = static_cast<int>(ns);
  p.persistent = 1;
  return fixed + ns * stage;
}

cudaError_t launch_tensor_gather2(const RowGemmParams& p, int dtype, size_t smem_bytes, cudaStream_t st) {
  const bool nc = (p.w_layout == EGS_W_NC);
  TensorMap3 m;
  const unsigned long long dims[3] = {static_cast<unsigned long long>(nc ? p.C : p.N), static_cast<unsigned long long>(nc ? p.N : p.C),
                                      static_cast<unsigned long long>(p.E)};
  const unsigned box[3] = {64u, nc ? static_cast<unsigned>(p.BN / 2) : 64u, 1u};
  if (!encode_tensor_map_16bit(&m, p.W, dims, box)) return cudaErrorInvalidValue;
  const long long ntiles = static_cast<long long>((p.M + 2 * kG2Rows - 1) / (2 * kG2Rows)) * p.E;      // 512 expert rows each
  dim3 grid(2 * static_cast<unsigned>(ntiles < kG2Pairs ? ntiles : kG2Pairs));
  dim3 block(kG2Threads);
  static thread_local int optin_device = -1;
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  if (optin_device != dev) {
    const int lim = static_cast<int>(kG2SmemMax);
    err = cudaFuncSetAttribute(tensor_gather2_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim);
    if (err == cudaSuccess) err = cudaFuncSetAttribute(tensor_gather2_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim);
    if (err != cudaSuccess) return err;
    optin_device = dev;
  }
  if (dtype == EGS_F16) tensor_gather2_kernel<__half><<<grid, block, smem_bytes, st>>>(p, m);
  else tensor_gather2_kernel<__nv_bfloat16><<<grid, block, smem_bytes, st>>>(p, m);
  count_launch();
  return cudaGetLastError();
}

}  // namespace egs
