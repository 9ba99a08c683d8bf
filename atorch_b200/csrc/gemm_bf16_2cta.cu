// bf16 GEMM for sm_100a with CTA pairs: tcgen05.mma.cta_group::2, 256 x 256 output tile per pair.
//
//   C[M,N] (+)= alpha * A[M,K] * B[N,K]^T (+ bias)        same contract as gemm_bf16.cu
//
// Two CTAs on neighbouring SMs form a cluster. Each loads its own 128 rows of A and its own 128
// rows (half) of the B tile, 32 KB per stage instead of 48 KB, so the ring is 6 stages deep and
// every byte of B is fetched once per pair. The leader CTA (cluster rank 0) issues the MMAs for
// both SMs; each CTA's tensor memory receives its own 128 rows of the 256 x 256 accumulator and
// each CTA runs its own epilogue. No TMA copy here is shared between CTAs: every load lands in
// the shared memory of the CTA that issued it and only its completion is signalled to the leader.
//
// Barrier protocol (per stage s, per accumulator a):
//   full[s]    leader only : leader's producer arrives with the pair's byte count (64 KB); the TMA
//                            loads of BOTH CTAs complete on it
//   empty[s]   both CTAs   : tcgen05.commit from the leader arrives on both
//   tfull[a]   both CTAs   : tcgen05.commit from the leader arrives on both
//   tempty[a]  leader only : the 4 epilogue warps of both CTAs arrive (8 arrivals)
//
// Fused with collectives over NVLink (tensor parallelism with sequence-sharded activations):
//   all-gather -> GEMM   the rows of A arrive shard by shard in a local buffer (copy engines pulling the
//                        peers' shards); `Gate` carries one arrival flag per shard, the TMA producer of a
//                        tile waits (bounded) for the flag of the shard that holds its rows, and the tiles
//                        are visited starting with this rank's own shard, so the math starts at once and
//                        the transfers hide behind it
//   GEMM -> reduce-scatter  the epilogue adds every output row into the fp32 accumulation buffer of the
//                        rank that owns the row (`red.add.f32` on peer pointers): no partial-sum tensor, no
//                        separate collective, the reduction traffic overlaps the remaining tiles
#include <cstdlib>
#include <mutex>

#include "common.cuh"

namespace {
using namespace atb;

constexpr int BM = 128;   // rows of A per CTA (256 per pair)
constexpr int BK = 64;
constexpr int A_BYTES = BM * BK * 2;

// BN = accumulator columns of the pair's tile (256 or 128); each CTA loads BN/2 rows of B.
// The narrower tile exists for wave quantisation: 256 tiles of 256x256 fill 74 CTA pairs 3.46 times
// (4 waves, 86 % busy), the same problem in 256x128 tiles takes 7 waves of half the length (99 %).
template <int BN>
struct Cfg {
  static constexpr int BNH = BN / 2;
  static constexpr int STAGES = BN == 256 ? 6 : 8;
  static constexpr int B_BYTES = BNH * BK * 2;
  static constexpr int BAR_OFF = STAGES * (A_BYTES + B_BYTES);
  static constexpr int TQ = 4;                     // tile-id ring of the dynamic scheduler
  static constexpr int SMEM_TOTAL = BAR_OFF + (2 * STAGES + 4 + 2 * TQ) * 8 + 16 + TQ * 4 + 1024;
};

struct Epi {
  void* C;
  const void* bias;
  long long ldc;
  float alpha;
  int out_fp32, accumulate;
  const void* residual;  // optional bf16 [M, N] added in the epilogue (pitch ldr); bf16 output only
  long long ldr;
  // reduce-scatter epilogue (rs_rows > 0): row r goes to rank r / rs_rows, as fp32 atomic adds into
  // rs_base[rank] + (r % rs_rows) * ldc + column; C is not written
  float* rs_base[8];
  int rs_rows;
  // gated (SwiGLU) epilogue: B is the fused gate|up weight [2 N, K] (K-major); a tile pairs gate rows
  // [f0, f0 + BN/2) (CTA 0's half of B) with up rows [N + f0, ...) (CTA 1's half), so that accumulator columns c
  // and BN/2 + c belong to the same output feature, and C[:, f0 + c] = silu(gate) * up is written as bf16. With
  // gu_out != null the bf16 gate and up values are stored too ([M, 2 N], pitch ldgu) for the backward pass.
  int gated;
  void* gu_out;
  long long ldgu;
};

// Arrival flags of the A operand (all-gather -> GEMM): rows [g * rows, (g + 1) * rows) are in place once
// flags[g] >= epoch (wrap-safe). rot = first tile row to visit (this rank's own shard).
// on_b: the flags describe rows of B (a weight gathered from row shards) instead of rows of A; rot then counts
// tile columns.
struct Gate {
  const unsigned int* flags;
  unsigned int epoch;
  int rows, rot;
  int on_b;
};

__device__ unsigned long long g_gate_wait_ns = ATB_WAIT_LIMIT_NS;

ATB_DEVICE bool gate_wait(const Gate& gate, int row_lo, int row_hi, volatile int* abort_flag, int* status) {
  for (int g = row_lo / gate.rows; g <= (row_hi - 1) / gate.rows; ++g) {
    const unsigned int* f = gate.flags + g;
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
    if ((int)(v - gate.epoch) >= 0) continue;
    const unsigned long long limit = g_gate_wait_ns;
    const uint64_t t0 = globaltimer_ns();
    while (true) {
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
      if ((int)(v - gate.epoch) >= 0) break;
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > limit) {
        *abort_flag = 1;
        if (status) atomicCAS(status, 0, (int)ATB_ERR_PEER_TIMEOUT);
        return false;
      }
      __nanosleep(200);
    }
  }
  // the rows were written by the copy engines / generic proxy; the loads that follow go through TMA
  asm volatile("fence.proxy.async.global;" ::: "memory");
  return true;
}

// Row groups with device-resident fill counts (mixture-of-experts buffers: `rows` slots per group, only
// the first counts[g] hold data and the rest is zero).
//   m_rows > 0 : rows of A / C form groups of m_rows (a multiple of 256). A tile that starts at or beyond
//                its group's count does no loads and no MMAs; its output is written as zeros.
//   b_rows > 0 : every bm_rows rows of A / C (a multiple of 256; one expert's slots from all sources)
//                multiply with their own B: the B tile coordinate is shifted by (m0 / bm_rows) * b_rows
//                along B's row axis (N for K-major B, K for MN-major B): B is [n_b * b_rows, ...].
//   k_rows > 0 : the reduction dim forms groups of k_rows (a multiple of 64); k-blocks at or beyond their
//                group's count are skipped (both operands are zero there).
struct Groups {
  const int* counts;
  int m_rows, b_rows, k_rows, bm_rows;
};

ATB_DEVICE uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
ATB_DEVICE void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `ptr` (a shared::cta pointer of this CTA) in CTA `rank` of the cluster
ATB_DEVICE uint32_t map_to_cta(const void* ptr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(ptr)), "r"(rank));
  return r;
}
// TMA load into this CTA's shared memory whose completion is counted on a barrier given by its
// shared::cluster address (the leader's).
ATB_DEVICE void tma_load_2d_pair(void* smem_dst, const CUtensorMap* tm, uint32_t bar_cluster_addr, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], "
      "[%2];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(tm)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
// Dynamic tile scheduling: tiles are handed out by an atomic counter instead of a fixed stride, so that a CTA pair
// that shares its SMs with another kernel (a reduce-scatter or copy kernel of the communication streams takes part
// of the SM's path to L2, on which this kernel's operand loads depend) simply takes fewer tiles, instead of making
// the whole launch wait for it. counters[0] = next tile, counters[1] = pairs that have finished; both are zero
// between launches (the pair that finishes last clears them).
struct Sched {
  int* counters;   // nullptr: static schedule (tile = pair + i * pairs)
};

ATB_DEVICE void st_remote_u32(uint32_t cluster_addr, uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
// Wait on a barrier whose phase is completed by an arrive of another CTA of the cluster that published data with it.
ATB_DEVICE bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status) {
  uint64_t t0 = 0;
  uint32_t spins = 0;
  while (true) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    if (ok) return true;
    if ((++spins & 0x3ff) == 0) {
      if (t0 == 0) t0 = globaltimer_ns();
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > ATB_WAIT_LIMIT_NS) {
        *abort_flag = 1;
        if (status) atomicCAS(status, 0, (int)ATB_ERR_WAIT_TIMEOUT);
        return false;
      }
    }
  }
}
ATB_DEVICE void mbar_arrive_remote(uint32_t bar_cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}

template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(192, 1)
gemm_bf16_2cta_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, Epi ep, int M,
                      int N, int K, Groups grp, Gate gate, Sched sched, int* status) {
  constexpr int BNH = Cfg<BN>::BNH, STAGES = Cfg<BN>::STAGES, B_BYTES = Cfg<BN>::B_BYTES,
                BAR_OFF = Cfg<BN>::BAR_OFF;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + BAR_OFF);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  constexpr int TQ = Cfg<BN>::TQ;
  uint64_t* tq_full = tempty + 2;
  uint64_t* tq_empty = tq_full + TQ;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tq_empty + TQ);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* tq_tile = reinterpret_cast<volatile int*>(tmem_slot + 4);   // [TQ] tile ids (-1: no more tiles)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  // both CTAs of a pair read the same word, so they take the same decision
  const bool skip = status != nullptr && *reinterpret_cast<volatile int*>(status) != 0;

  const int tiles_m = (M + 2 * BM - 1) / (2 * BM);
  const int tile_cols = ep.gated ? BN / 2 : BN;      // output columns per tile
  const int tiles_n = (N + tile_cols - 1) / tile_cols;
  const int num_tiles = skip ? 0 : tiles_m * tiles_n;
  const int num_kb = (K + BK - 1) / BK;
  const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;
  constexpr int BAND = 8;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    mbar_init(&tfull[0], 1);
    mbar_init(&tfull[1], 1);
    mbar_init(&tempty[0], 8);
    mbar_init(&tempty[1], 8);
    for (int i = 0; i < TQ; ++i) {
      mbar_init(&tq_full[i], 1);
      mbar_init(&tq_empty[i], 10);   // leader: MMA thread + 4 epilogue warps; partner: producer + 4 epilogue warps
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc<2>(tmem_slot, 2 * BN);
    tmem_relinquish<2>();
  }
  tc_fence_before();
  cluster_sync_all();  // barriers of both CTAs initialised and visible before any remote arrive
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // identical decisions in every role: which tiles and which k-blocks carry data
  auto tile_active = [&](int m0) -> bool {
    if (grp.counts == nullptr) return true;
    if (grp.m_rows > 0) {
      const int g = m0 / grp.m_rows;
      if (m0 - g * grp.m_rows >= grp.counts[g]) return false;
    }
    if (grp.k_rows > 0) {   // nothing to reduce over at all?
      const int ng = (K + grp.k_rows - 1) / grp.k_rows;
      bool any = false;
      for (int g = 0; g < ng; ++g) any |= grp.counts[g] > 0;
      return any;
    }
    return true;
  };
  auto kb_active = [&](int kb) -> bool {
    if (grp.counts == nullptr || grp.k_rows <= 0) return true;
    const int k0 = kb * BK, g = k0 / grp.k_rows;
    return k0 - g * grp.k_rows < grp.counts[g];
  };

  auto tile_coords = [&](int tile, int& m0, int& n0) {
    const int band_tiles = BAND * tiles_n;
    const int band = tile / band_tiles;
    const int rem = tile - band * band_tiles;
    const int rows_in_band = min(BAND, tiles_m - band * BAND);
    int tn = rem / rows_in_band;
    int tm = band * BAND + (rem - tn * rows_in_band);
    if (gate.rot > 0) {          // start with the rows that are already here
      if (gate.on_b) {
        tn += gate.rot;
        if (tn >= tiles_n) tn -= tiles_n;
      } else {
        tm += gate.rot;
        if (tm >= tiles_m) tm -= tiles_m;
      }
    }
    m0 = tm * 2 * BM;
    n0 = tn * tile_cols;
  };

  // The idx-th tile of this pair, the same number in every role of both CTAs. Static: a fixed stride. Dynamic: the
  // leader's producer thread draws it from the global counter and publishes it through a ring of tile ids in the
  // shared memory of both CTAs; every other role reads it there and frees the slot.
  const bool dyn = sched.counters != nullptr;
  auto static_tile = [&](int idx) -> int {
    const int t = cluster_id + idx * num_clusters;
    return t < num_tiles ? t : -1;
  };
  auto publish_tile = [&](int idx, int t) -> bool {          // leader's producer thread
    const int slot = idx % TQ;
    if (!mbar_wait(&tq_empty[slot], ((idx / TQ) & 1) ^ 1, abort_flag, status)) return false;
    tq_tile[slot] = t;
    st_remote_u32(map_to_cta(const_cast<int*>(&tq_tile[slot]), 1), (uint32_t)t);
    mbar_arrive(&tq_full[slot]);
    mbar_arrive_remote(map_to_cta(&tq_full[slot], 1));       // release.cluster: orders the store above
    return true;
  };
  auto read_tile = [&](int idx) -> int {                      // any other role (one thread, or all lanes of a warp)
    if (!dyn) return static_tile(idx);
    const int slot = idx % TQ;
    if (!mbar_wait_cluster(&tq_full[slot], (idx / TQ) & 1, abort_flag, status)) return -1;
    return tq_tile[slot];
  };
  auto free_tile_slot = [&](int idx) {                        // one thread per consumer, after read_tile
    if (dyn) mbar_arrive_remote(map_to_cta(&tq_empty[idx % TQ], 0));
  };

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      int drawn = (dyn && leader) ? atomicAdd(&sched.counters[0], 1) : 0;
      for (int idx = 0;; ++idx) {
        int tile;
        if (dyn && leader) {
          tile = drawn < num_tiles ? drawn : -1;
          if (tile >= 0) drawn = atomicAdd(&sched.counters[0], 1);     // the next one, fetched under this tile's loads
          if (!publish_tile(idx, tile)) goto producer_done;
          if (tile < 0) {      // every pair draws exactly one number past the end; the last pair to do so resets
            if (atomicAdd(&sched.counters[1], 1) == num_clusters - 1) {
              sched.counters[0] = 0;
              sched.counters[1] = 0;
              __threadfence();
            }
          }
        } else {
          tile = read_tile(idx);
          free_tile_slot(idx);
        }
        if (tile < 0) break;
        int m0, n0;
        tile_coords(tile, m0, n0);
        if (!tile_active(m0)) continue;
        const int am0 = m0 + (int)rank * BM;   // this CTA's rows of A
        const int bshift = grp.b_rows > 0 ? (m0 / grp.bm_rows) * grp.b_rows : 0;   // this expert's own B
        // this CTA's rows of B (gated: CTA 0 takes gate rows, CTA 1 the up rows of the same features)
        const int bn0 = ep.gated ? n0 + (int)rank * N : n0 + (int)rank * BNH + (B_MN ? 0 : bshift);
        const int bk0 = B_MN ? bshift : 0;
        if (gate.flags != nullptr) {
          const bool here = gate.on_b ? gate_wait(gate, min(bn0, N - 1), min(bn0 + BNH, N), abort_flag, status)
                                      : gate_wait(gate, am0, min(am0 + BM, M), abort_flag, status);
          if (!here) goto producer_done;
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!kb_active(kb)) continue;
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, status)) goto producer_done;
          if (leader) mbar_expect_tx(&full[s], 2 * (A_BYTES + B_BYTES));
          const uint32_t bar = map_to_cta(&full[s], 0);
          uint8_t* a_dst = sA + s * A_BYTES;
          uint8_t* b_dst = sB + s * B_BYTES;
          if constexpr (!A_MN) {
            tma_load_2d_pair(a_dst, &tmA, bar, kb * BK, am0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d_pair(a_dst + j * 8192, &tmA, bar, am0 + j * 64, kb * BK);
          }
          if constexpr (!B_MN) {
            tma_load_2d_pair(b_dst, &tmB, bar, kb * BK, bn0);
          } else {
#pragma unroll
            for (int j = 0; j < BNH / 64; ++j)
              tma_load_2d_pair(b_dst + j * 8192, &tmB, bar, bn0 + j * 64, bk0 + kb * BK);
          }
          ++it;
        }
      }
    }
  producer_done:;
  } else if (warp == 1) {
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = umma_idesc(2 * BM, BN, 1, 1, A_MN, B_MN);
      uint32_t it = 0;
      int local = 0;
      for (int idx = 0;; ++idx) {
        const int tile = read_tile(idx);
        free_tile_slot(idx);
        if (tile < 0) break;
        {
          int m0, n0;
          tile_coords(tile, m0, n0);
          if (!tile_active(m0)) continue;
        }
        const int acc = local & 1;
        const uint32_t acc_ph = (local >> 1) & 1;
        if (!mbar_wait(&tempty[acc], acc_ph ^ 1, abort_flag, status)) goto mma_done;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        bool first_kb = true;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!kb_active(kb)) continue;
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&full[s], ph, abort_flag, status)) goto mma_done;
          tc_fence_after();
          const uint32_t a_addr = smem_u32(sA + s * A_BYTES);
          const uint32_t b_addr = smem_u32(sB + s * B_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t adesc = A_MN ? umma_desc_sw128(a_addr + k * 2048, 8192, 1024)
                                        : umma_desc_sw128(a_addr + k * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? umma_desc_sw128(b_addr + k * 2048, 8192, 1024)
                                        : umma_desc_sw128(b_addr + k * 32, 16, 1024);
            umma_f16<2>(d_tmem, adesc, bdesc, idesc, (first_kb && k == 0) ? 0u : 1u);
          }
          first_kb = false;
          umma_commit_cg2(smem_u32(&empty[s]));
          umma_commit_cg2(map_to_cta(&empty[s], 1));
          ++it;
        }
        umma_commit_cg2(smem_u32(&tfull[acc]));
        umma_commit_cg2(map_to_cta(&tfull[acc], 1));
        ++local;
      }
    }
  mma_done:;
  } else {
    const int q = warp & 3;
    int local = 0;
    const uint32_t tempty_leader[2] = {map_to_cta(&tempty[0], 0), map_to_cta(&tempty[1], 0)};
    for (int idx = 0;; ++idx) {
      const int tile = __shfl_sync(0xffffffffu, read_tile(idx), 0);
      __syncwarp();
      if (lane == 0) free_tile_slot(idx);
      if (tile < 0) break;
      int m0, n0;
      tile_coords(tile, m0, n0);
      if (!tile_active(m0)) {
        // an empty tile: its output is all zeros (left alone when accumulating)
        const int zrow = m0 + (int)rank * BM + q * 32 + lane;
        if (!ep.accumulate && ep.rs_rows <= 0 && zrow < M) {
          for (int c = 0; c < BN; c += 8) {
            if (n0 + c >= N) break;
            if (ep.out_fp32) {
              float* z = reinterpret_cast<float*>(ep.C) + (long long)zrow * ep.ldc + n0 + c;
              *reinterpret_cast<float4*>(z) = make_float4(0.f, 0.f, 0.f, 0.f);
              *reinterpret_cast<float4*>(z + 4) = make_float4(0.f, 0.f, 0.f, 0.f);
            } else {
              *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(ep.C) + (long long)zrow * ep.ldc + n0 + c) =
                  make_uint4(0u, 0u, 0u, 0u);
            }
          }
        }
        continue;
      }
      const int acc = local & 1;
      const uint32_t acc_ph = (local >> 1) & 1;
      if (!__all_sync(0xffffffffu, mbar_wait(&tfull[acc], acc_ph, abort_flag, status))) break;
      tc_fence_after();
      const int row = m0 + (int)rank * BM + q * 32 + lane;
      const uint32_t t_addr = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN;
      if (ep.gated) {
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          uint32_t g[32], u[32];
          tmem_ld_32x32(t_addr + c * 32, g);
          tmem_ld_32x32(t_addr + BN / 2 + c * 32, u);
          tmem_ld_wait();
          const int col0 = n0 + c * 32;
          if (row < M && col0 < N) {
            __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(ep.C) + (long long)row * ep.ldc + col0;
            __nv_bfloat16* grow = ep.gu_out == nullptr ? nullptr
                : reinterpret_cast<__nv_bfloat16*>(ep.gu_out) + (long long)row * ep.ldgu + col0;
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              if (col0 + i < N) {
                uint32_t gp[4], up[4], op[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  // round to bf16 first: the same values and the same formula as the separate SwiGLU kernel
                  gp[j] = pack_bf16x2(__uint_as_float(g[i + 2 * j]), __uint_as_float(g[i + 2 * j + 1]));
                  up[j] = pack_bf16x2(__uint_as_float(u[i + 2 * j]), __uint_as_float(u[i + 2 * j + 1]));
                  const float2 a = unpack_bf16x2(gp[j]), b = unpack_bf16x2(up[j]);
                  op[j] = pack_bf16x2(a.x / (1.f + __expf(-a.x)) * b.x, a.y / (1.f + __expf(-a.y)) * b.y);
                }
                *reinterpret_cast<uint4*>(crow + i) = make_uint4(op[0], op[1], op[2], op[3]);
                if (grow != nullptr) {
                  *reinterpret_cast<uint4*>(grow + i) = make_uint4(gp[0], gp[1], gp[2], gp[3]);
                  *reinterpret_cast<uint4*>(grow + N + i) = make_uint4(up[0], up[1], up[2], up[3]);
                }
              }
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_remote(tempty_leader[acc]);
        ++local;
        continue;
      }
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(t_addr + c * 32, r);
        tmem_ld_wait();
        const int col0 = n0 + c * 32;
        if (row < M && col0 < N) {
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * ep.alpha;
          if (ep.bias != nullptr) {
            const __nv_bfloat16* bias = reinterpret_cast<const __nv_bfloat16*>(ep.bias);
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (col0 + i < N) v[i] += __bfloat162float(bias[col0 + i]);
          }
          if (ep.rs_rows > 0) {
            const int owner = row / ep.rs_rows;
            float* crow = ep.rs_base[owner] + (long long)(row - owner * ep.rs_rows) * ep.ldc + col0;
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              if (col0 + i < N)
                asm volatile("red.relaxed.sys.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(crow + i), "f"(v[i]),
                             "f"(v[i + 1]), "f"(v[i + 2]), "f"(v[i + 3])
                             : "memory");
            }
          } else if (ep.out_fp32) {
            float* crow = reinterpret_cast<float*>(ep.C) + (long long)row * ep.ldc + col0;
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              if (col0 + i < N) {
                float4 o = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
                if (ep.accumulate) {
                  const float4 old = *reinterpret_cast<const float4*>(crow + i);
                  o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                }
                *reinterpret_cast<float4*>(crow + i) = o;
              }
            }
          } else {
            __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(ep.C) + (long long)row * ep.ldc + col0;
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              if (col0 + i < N) {
                if (ep.accumulate) {
                  const uint4 old = *reinterpret_cast<const uint4*>(crow + i);
                  const float2 o0 = unpack_bf16x2(old.x), o1 = unpack_bf16x2(old.y), o2 = unpack_bf16x2(old.z),
                               o3 = unpack_bf16x2(old.w);
                  v[i] += o0.x; v[i + 1] += o0.y; v[i + 2] += o1.x; v[i + 3] += o1.y;
                  v[i + 4] += o2.x; v[i + 5] += o2.y; v[i + 6] += o3.x; v[i + 7] += o3.y;
                }
                if (ep.residual != nullptr) {
                  const uint4 rr = *reinterpret_cast<const uint4*>(
                      reinterpret_cast<const __nv_bfloat16*>(ep.residual) + (long long)row * ep.ldr + col0 + i);
                  const float2 r0 = unpack_bf16x2(rr.x), r1 = unpack_bf16x2(rr.y), r2 = unpack_bf16x2(rr.z),
                               r3 = unpack_bf16x2(rr.w);
                  v[i] += r0.x; v[i + 1] += r0.y; v[i + 2] += r1.x; v[i + 3] += r1.y;
                  v[i + 4] += r2.x; v[i + 5] += r2.y; v[i + 6] += r3.x; v[i + 7] += r3.y;
                }
                uint4 o;
                o.x = pack_bf16x2(v[i], v[i + 1]);
                o.y = pack_bf16x2(v[i + 2], v[i + 3]);
                o.z = pack_bf16x2(v[i + 4], v[i + 5]);
                o.w = pack_bf16x2(v[i + 6], v[i + 7]);
                *reinterpret_cast<uint4*>(crow + i) = o;
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(tempty_leader[acc]);
      ++local;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  // neither CTA may leave (or free tensor memory) while its partner can still signal its barriers
  // or while the leader's MMAs can still write into the partner's tensor memory
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<2>(tmem_base, 2 * BN);
  }
}

int g_sms = 0;
int sm_count() {
  if (g_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_sms <= 0) g_sms = 148;
  }
  return g_sms;
}

// Counters of the dynamic tile scheduler: one pair per (device, stream), because launches on different streams can
// overlap. Allocated and zeroed on first use (never during a stream capture: such launches use the static schedule).
struct SchedWs {
  int dev;
  cudaStream_t stream;
  int* counters;
};
constexpr int SCHED_MAX_STREAMS = 16;
SchedWs g_sched_ws[SCHED_MAX_STREAMS];
int g_sched_n = 0;
int g_dynamic = -1;      // -1: read ATB_GEMM_DYNAMIC on first use (default on)
std::mutex g_sched_mu;

int* sched_counters(cudaStream_t stream) {
  std::lock_guard<std::mutex> lock(g_sched_mu);
  int dev = 0;
  cudaGetDevice(&dev);
  for (int i = 0; i < g_sched_n; ++i)
    if (g_sched_ws[i].dev == dev && g_sched_ws[i].stream == stream) return g_sched_ws[i].counters;
  if (g_sched_n >= SCHED_MAX_STREAMS) return nullptr;
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) {
    cudaGetLastError();
    return nullptr;
  }
  void* p = nullptr;
  if (cudaMalloc(&p, 256) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  if (cudaMemsetAsync(p, 0, 256, stream) != cudaSuccess) {
    cudaGetLastError();
    cudaFree(p);
    return nullptr;
  }
  g_sched_ws[g_sched_n++] = SchedWs{dev, stream, reinterpret_cast<int*>(p)};
  return reinterpret_cast<int*>(p);
}

template <int BN, bool A_MN, bool B_MN>
int launch(const void* A, const void* B, const Epi& ep, int M, int N, int K, long long lda, long long ldb,
           int max_ctas, const Groups& grp, int b_extent_rows, const Gate& gate, cudaStream_t stream, int* status) {
  CUtensorMap tmA, tmB;
  bool ok;
  if (!A_MN)
    ok = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, lda, BM, BK, CU_TENSOR_MAP_SWIZZLE_128B);
  else
    ok = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, M, lda, BK, 64, CU_TENSOR_MAP_SWIZZLE_128B);
  if (!ok) return -2;
  // with per-group B the tensor map spans all groups' weights (b_extent_rows rows)
  if (!B_MN)
    ok = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, b_extent_rows > 0 ? b_extent_rows : N, K, ldb,
                      Cfg<BN>::BNH, BK, CU_TENSOR_MAP_SWIZZLE_128B);
  else
    ok = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, b_extent_rows > 0 ? b_extent_rows : K, N, ldb, BK,
                      64, CU_TENSOR_MAP_SWIZZLE_128B);
  if (!ok) return -3;
  auto kern = gemm_bf16_2cta_kernel<BN, A_MN, B_MN>;
  constexpr int SMEM_TOTAL = Cfg<BN>::SMEM_TOTAL;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL) != cudaSuccess) return -4;
    attr_set = true;
  }
  const int tile_cols = ep.gated ? BN / 2 : BN;
  const int tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((N + tile_cols - 1) / tile_cols);
  int clusters = sm_count() / 2;
  if (tiles < clusters) clusters = tiles;
  if (max_ctas > 0 && clusters > max_ctas / 2) clusters = max_ctas / 2 > 0 ? max_ctas / 2 : 1;
  // dynamic tile scheduling for plain launches with more tiles than CTA pairs (see Sched)
  Sched sched{nullptr};
  if (g_dynamic < 0) {
    const char* e = getenv("ATB_GEMM_DYNAMIC");
    g_dynamic = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  if (g_dynamic > 0 && tiles > clusters && grp.counts == nullptr && grp.b_rows == 0 && gate.flags == nullptr)
    sched.counters = sched_counters(stream);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * clusters, 1, 1);
  cfg.blockDim = dim3(192, 1, 1);
  cfg.dynamicSmemBytes = SMEM_TOTAL;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tmA, tmB, ep, M, N, K, grp, gate, sched, status);
  return e == cudaSuccess ? 0 : -5;
}

// extra arguments of the next launch of this host thread (set and cleared by atb_gemm_bf16_2cta_fused)
struct FusedArgs {
  bool active;
  Gate gate;
  float* rs_base[8];
  int rs_rows;
};
thread_local FusedArgs g_fused_args = {false, {nullptr, 0u, 1, 0}, {nullptr}, 0};

}  // namespace

// Same arguments as atb_gemm_bf16 (gemm_bf16.cu) minus the tile choice, plus row groups (see Groups):
// `group_counts` int32 device array or null with m_group_rows (multiple of 256) and / or k_group_rows
// (multiple of 64); b_group_rows > 0: every bm_group_rows rows of A use their own B out of n_b stacked
// ones, as described there. Best for M, N >= 256.
extern "C" int atb_gemm_bf16_2cta_grouped(const void* A, const void* B, void* C, const void* bias, int M, int N, int K,
                                          long long lda, long long ldb, long long ldc, int a_mn_major, int b_mn_major,
                                          int out_fp32, int accumulate, float alpha, int tile_n, int max_ctas,
                                          const void* residual, long long ldr, const int* group_counts,
                                          int m_group_rows, int k_group_rows, int b_group_rows, int bm_group_rows,
                                          int n_b, void* stream, int* status) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((N & 7) || (lda & 7) || (ldb & 7) || (ldc & 3) || (!out_fp32 && (ldc & 7))) return -1;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15)
    return -1;
  if (residual != nullptr && (out_fp32 || (ldr & 7) || (reinterpret_cast<uintptr_t>(residual) & 15))) return -1;
  Groups grp{nullptr, 0, 0, 0, 0};
  int b_extent = 0;
  if ((m_group_rows % 256) || (k_group_rows % 64) || (bm_group_rows % 256) || m_group_rows < 0 ||
      k_group_rows < 0 || b_group_rows < 0)
    return -1;
  if (group_counts != nullptr) {
    grp.counts = group_counts;
    grp.m_rows = m_group_rows;
    grp.k_rows = k_group_rows;
  }
  if (b_group_rows > 0) {
    if (bm_group_rows <= 0 || n_b <= 0) return -1;
    grp.b_rows = b_group_rows;
    grp.bm_rows = bm_group_rows;
    b_extent = n_b * b_group_rows;
  }
  Epi ep{C, bias, ldc, alpha, out_fp32, accumulate, residual, ldr, {nullptr}, 0, 0, nullptr, 0};
  Gate gate{nullptr, 0u, 1, 0};
  if (g_fused_args.active) {   // set by atb_gemm_bf16_2cta_fused for this one launch
    gate = g_fused_args.gate;
    for (int i = 0; i < 8; ++i) ep.rs_base[i] = g_fused_args.rs_base[i];
    ep.rs_rows = g_fused_args.rs_rows;
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  // The 256-wide tile is the default. The 128-wide one fills the last wave better (256 tiles of 256x256
  // occupy 74 CTA pairs for 4 waves at 86 %), but measured 1.5x slower per FLOP on B200: its 256-cycle
  // stages leave the single MMA-issuing thread no slack. It stays selectable with tile_n = 128.
  const bool narrow = tile_n == 128;
#define ATB_PAIR_DISPATCH(BN_)                                                                                     \
  do {                                                                                                             \
    if (!a_mn_major && !b_mn_major)                                                                                \
      return launch<BN_, false, false>(A, B, ep, M, N, K, lda, ldb, max_ctas, grp, b_extent, gate, st, status);          \
    if (!a_mn_major && b_mn_major)                                                                                 \
      return launch<BN_, false, true>(A, B, ep, M, N, K, lda, ldb, max_ctas, grp, b_extent, gate, st, status);           \
    if (a_mn_major && b_mn_major)                                                                                  \
      return launch<BN_, true, true>(A, B, ep, M, N, K, lda, ldb, max_ctas, grp, b_extent, gate, st, status);            \
    return launch<BN_, true, false>(A, B, ep, M, N, K, lda, ldb, max_ctas, grp, b_extent, gate, st, status);             \
  } while (0)
  if (narrow) ATB_PAIR_DISPATCH(128);
  ATB_PAIR_DISPATCH(256);
#undef ATB_PAIR_DISPATCH
}

extern "C" int atb_gemm_bf16_2cta(const void* A, const void* B, void* C, const void* bias, int M, int N, int K,
                                  long long lda, long long ldb, long long ldc, int a_mn_major, int b_mn_major,
                                  int out_fp32, int accumulate, float alpha, int tile_n, int max_ctas,
                                  const void* residual, long long ldr, void* stream, int* status) {
  return atb_gemm_bf16_2cta_grouped(A, B, C, bias, M, N, K, lda, ldb, ldc, a_mn_major, b_mn_major, out_fp32,
                                    accumulate, alpha, tile_n, max_ctas, residual, ldr, nullptr, 0, 0, 0, 0, 0, stream,
                                    status);
}

// act[M, F] = silu(x Wg^T) * (x Wu^T) for the fused weight W = [Wg; Wu] ([2 F, K], K-major, pitch ldb): the GEMM with
// the gated epilogue (see Epi). gu_out (optional, [M, 2 F] bf16, pitch ldgu) receives the gate and up values the
// backward pass needs. F % 8 == 0; x is [M, K] K-major with pitch lda.
extern "C" int atb_gemm_bf16_2cta_swiglu(const void* A, const void* B, void* act, void* gu_out, int M, int F, int K,
                                         long long lda, long long ldb, long long ld_act, long long ldgu, void* stream,
                                         int* status) {
  if (M <= 0 || F <= 0 || K <= 0) return 0;
  if ((F & 7) || (lda & 7) || (ldb & 7) || (ld_act & 7) || (gu_out != nullptr && (ldgu & 7))) return -1;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(act) |
       reinterpret_cast<uintptr_t>(gu_out)) & 15)
    return -1;
  Epi ep{act, nullptr, ld_act, 1.f, 0, 0, nullptr, 0, {nullptr}, 0, 1, gu_out, ldgu};
  Groups grp{nullptr, 0, 0, 0, 0};
  Gate gate{nullptr, 0u, 1, 0};
  return launch<256, false, false>(A, B, ep, M, F, K, lda, ldb, 0, grp, 2 * F, gate,
                                   reinterpret_cast<cudaStream_t>(stream), status);
}

// Weight all-gather -> GEMM (a linear layer whose weight is sharded by rows over the ranks): C = A B^T with
// B [N, K] K-major arriving in shards of gate_rows rows (a multiple of 128); shard g is in place once
// gate_flags[g] >= gate_epoch. Tiles start at column gate_first_row (a multiple of 256: this rank's own shard).
extern "C" int atb_gemm_bf16_2cta_wgather(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                                          long long ldb, long long ldc, const unsigned int* gate_flags,
                                          unsigned int gate_epoch, int gate_rows, int gate_first_row, void* stream,
                                          int* status) {
  if (gate_flags == nullptr || gate_rows <= 0 || (gate_rows % 128) || gate_first_row < 0 || (gate_first_row % 256))
    return -1;
  FusedArgs fa = {true, {gate_flags, gate_epoch, gate_rows, gate_first_row / 256, 1}, {nullptr}, 0};
  g_fused_args = fa;
  const int rc = atb_gemm_bf16_2cta_grouped(A, B, C, nullptr, M, N, K, lda, ldb, ldc, 0, 0, 0, 0, 1.f, 0, 0, nullptr, 0,
                                            nullptr, 0, 0, 0, 0, 0, stream, status);
  g_fused_args.active = false;
  return rc;
}

// 1 / 0: hand tiles out dynamically or by a fixed stride (default: dynamic unless ATB_GEMM_DYNAMIC=0).
extern "C" void atb_gemm_set_dynamic(int on) { g_dynamic = on ? 1 : 0; }

// Upper bound of the arrival-flag waits of the all-gather -> GEMM form, in nanoseconds (default 2 s).
extern "C" int atb_set_gate_wait_ns(unsigned long long ns) {
  return cudaMemcpyToSymbol(g_gate_wait_ns, &ns, sizeof(ns)) == cudaSuccess ? 0 : -5;
}

// The GEMM fused with a collective (see the file header). On top of atb_gemm_bf16_2cta:
//   gate_flags != null : all-gather -> GEMM. A's rows arrive in shards of gate_rows rows (a multiple of 128);
//                        shard g is in place once gate_flags[g] >= gate_epoch; tiles start at row gate_first_row.
//   rs_ptrs != null    : GEMM -> reduce-scatter. rs_ptrs = `rs_world` device addresses of the ranks' fp32
//                        accumulation buffers [rs_rows, N] (pitch ldc); output row r is added into rank
//                        r / rs_rows' buffer. C may be null.
extern "C" int atb_gemm_bf16_2cta_fused(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                                        long long ldb, long long ldc, int a_mn_major, int b_mn_major, float alpha,
                                        const unsigned int* gate_flags, unsigned int gate_epoch, int gate_rows,
                                        int gate_first_row, const unsigned long long* rs_ptrs, int rs_world,
                                        int rs_rows, void* stream, int* status) {
  FusedArgs fa = {true, {nullptr, 0u, 1, 0}, {nullptr}, 0};
  if (gate_flags != nullptr) {
    if (gate_rows <= 0 || (gate_rows % 128) || a_mn_major || gate_first_row < 0 || (gate_first_row % 256)) return -1;
    fa.gate = Gate{gate_flags, gate_epoch, gate_rows, gate_first_row / 256};
  }
  void* c_arg = C;
  int out_fp32 = 0;
  if (rs_ptrs != nullptr) {
    if (rs_world < 1 || rs_world > 8 || rs_rows <= 0 || (long long)rs_rows * rs_world < M) return -1;
    for (int i = 0; i < rs_world; ++i) fa.rs_base[i] = reinterpret_cast<float*>(rs_ptrs[i]);
    fa.rs_rows = rs_rows;
    c_arg = fa.rs_base[0];     // only its alignment is checked; the epilogue never writes through it
    out_fp32 = 1;
  }
  g_fused_args = fa;
  const int rc = atb_gemm_bf16_2cta_grouped(A, B, c_arg, nullptr, M, N, K, lda, ldb, ldc, a_mn_major, b_mn_major,
                                            out_fp32, 0, alpha, 0, 0, nullptr, 0, nullptr, 0, 0, 0, 0, 0, stream,
                                            status);
  g_fused_args.active = false;
  return rc;
}
