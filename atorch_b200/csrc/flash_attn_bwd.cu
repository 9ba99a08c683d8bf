// Flash attention backward for sm_100a (head dim 128, bf16), tcgen05 + TMEM + TMA.
//
// One CTA per (128 keys, head, batch) walks the query blocks that can see its keys. Per query block:
//   S  = Q K^T,  dP = dO V^T                      2 x tcgen05.mma -> TMEM   (K-major operands)
//   P  = exp2(S c - lse),  dS = P (dP - delta) s    registers -> bf16 tiles in swizzled shared memory
//   dV += P^T dO,  dK += dS^T Q                    accumulate in TMEM across query blocks (MN-major operands)
//   dQ  = dS K                                      TMEM -> registers -> shared memory -> TMA reduce-add (fp32)
// A [rows][64] bf16 panel with 128-byte swizzle is at the same time a K-major tile of the matrix and
// an MN-major tile of its transpose, so P, dS, Q, dO and K are each stored once and read both ways.
// TMEM: S | dP | dV | dK = 4 x 128 columns; dQ reuses the dP columns.
//
// Warp 0 = TMA producer, warp 1 = MMA issuer and TMEM owner, warps 2..9 = element-wise work (thread
// (row r, half h) owns columns [64h, 64h+64) of row r). `delta = rowsum(dO * O)` comes from a
// small pre-pass; dQ is accumulated in fp32 and converted by a post-pass.
//
// Software pipeline over the query blocks (Q is double-buffered in shared memory):
//   tensor core, when P(i), dS(i) are in shared memory:  S(i+1) | dV(i) | dK(i) | dQ(i)
//   element-wise warps meanwhile:                        P(i+1) = exp2(S(i+1) c - lse)   (the exponentials)
//   then:  dQ(i) out of TMEM (red.add)  ->  tensor core: dP(i+1)  ->  dS(i+1), P(i+1) to shared memory
// so the exponentials and the loads of the next Q / dO tiles run under the three accumulating products.
// dQ(i) is staged in the shared memory of P and dS (free between the products of block i and the element-wise
// results of block i+1) and added to the fp32 accumulation buffer by four cp.reduce.async.bulk.tensor
// operations of one thread: the 64 KB of atomic adds per query block run in the TMA unit while the warps go on.
//
// Masks are per-row key intervals [lo, hi) as in the forward kernel.
#include "common.cuh"

namespace {
using namespace atb;

constexpr int BQ = 128, BKV = 128, HD = 128;
constexpr int PANEL = 128 * 64 * 2;
constexpr int TILE = 2 * PANEL;
constexpr int N_EW = 256;
constexpr int THREADS = 64 + N_EW;

struct BwdParams {
  const float* lse;    // [B, Hq, Sq]
  const float* delta;  // [B, Hq, Sq]
  float* dq_acc;       // [B, Sq, Hq, HD] fp32, zero-initialised
  __nv_bfloat16* dk;   // token-major, head h at columns [h*HD, h*HD+HD) of a row of pitch dkv_stride
  __nv_bfloat16* dv;
  long long dkv_stride;
  const int* row_lo;
  const int* row_hi;
  int B, Sq, Sk, Hq, Hkv, causal;
  float scale, scale_log2;
  int* status;
  DropParams drop;     // attention dropout of the forward pass (thr16 == 0: none)
  BiasParams bias;     // additive bias of the forward pass (ptr == nullptr: none); not differentiated
  float inv_scale;
};

struct SmemB {
  static constexpr int Q_OFF = 0;                 // two stages
  static constexpr int DO_OFF = Q_OFF + 2 * TILE;
  static constexpr int K_OFF = DO_OFF + TILE;
  static constexpr int V_OFF = K_OFF + TILE;
  static constexpr int P_OFF = V_OFF + TILE;
  static constexpr int DS_OFF = P_OFF + TILE;
  static constexpr int BAR_OFF = DS_OFF + TILE;  // 224 KB
  static constexpr int NBARS = 14;
  static constexpr int TOTAL = BAR_OFF + NBARS * 8 + 64 + 1024;
};
static_assert(SmemB::TOTAL <= 232448, "shared memory of the backward kernel exceeds 227 KB");

// Row of a query block as the element-wise thread sees it.
struct RowInfo {
  int i;          // global query row
  bool valid;     // inside the sequence and not fully masked
  int lo, hi;     // key interval
  float lse2, delta;
};

// WITH_DQ = false: key/value gradients only (the query gradient then comes from flash_attn_bwd_dq.cu): the
// dQ product, its staging and the reduce-add are compiled out and dP(i+1) follows dK(i) without a hand-shake.
// HDIM = 128 or 64 (64: one 64-column panel per Q / dO / K / V tile, 64-column dV / dK / dQ accumulators).
template <bool WITH_DQ, bool DROP = false, bool BIAS = false, int HDIM = 128>
__global__ void __launch_bounds__(THREADS, 1)
flash_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmdO,
                 const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                 const __grid_constant__ CUtensorMap tmdQ, BwdParams p) {
  using L = SmemB;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + L::Q_OFF;
  uint8_t* sdO = smem + L::DO_OFF;
  uint8_t* sK = smem + L::K_OFF;
  uint8_t* sV = smem + L::V_OFF;
  uint8_t* sP = smem + L::P_OFF;
  uint8_t* sdS = smem + L::DS_OFF;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* kv_full = bars;
  uint64_t* q_full = bars + 1;    // [2]
  uint64_t* q_free = bars + 3;    // [2]  dK(i) has read Q(i)
  uint64_t* do_full = bars + 5;
  uint64_t* do_free = bars + 6;   // dV(i) has read dO(i)
  uint64_t* s_full = bars + 7;    // S(i) is in TMEM
  uint64_t* dp_full = bars + 8;   // dP(i) is in TMEM
  uint64_t* pds_full = bars + 9;  // P(i), dS(i) are in shared memory; S(i), dP(i) have been read
  uint64_t* dq_full = bars + 10;  // dV(i), dK(i), dQ(i) are complete
  uint64_t* dp_free = bars + 11;  // dQ(i) has been read out of the dP columns
  uint64_t* stage_full = bars + 12;  // dQ(i) is staged in shared memory (all element-wise warps)
  uint64_t* stage_free = bars + 13;  // the TMA unit has read the staged dQ(i): P / dS may be written again
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + L::NBARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* q_range = const_cast<int*>(reinterpret_cast<volatile int*>(tmem_slot + 2));  // [2]: first, last+1 q block

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // a wait already ran out somewhere in this stream of work: do not start, so that a failing
  // launch ends after one wait limit instead of one per wave of CTAs
  if (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != 0) return;
  const int kb = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.Hq / p.Hkv);
  const int kv0 = kb * BKV;
  const int shift = p.Sk - p.Sq;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&q_free[i], 1);
    }
    mbar_init(do_full, 1);
    mbar_init(do_free, 1);
    mbar_init(s_full, 1);
    mbar_init(dp_full, 1);
    mbar_init(pds_full, N_EW / 32);
    mbar_init(dq_full, 1);
    mbar_init(dp_free, N_EW / 32);
    mbar_init(stage_full, N_EW / 32);
    mbar_init(stage_free, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc<1>(tmem_slot, 512);
    tmem_relinquish<1>();
  }
  if (warp == 2) {
    // query rows whose interval meets this key block
    int rmin = INT_MAX, rmax = -1;
    if (p.row_lo == nullptr && p.row_hi == nullptr) {
      if (lane == 0) {
        rmin = p.causal ? max(0, kv0 - shift) : 0;
        rmax = p.Sq - 1;
        if (rmin > rmax) { rmin = INT_MAX; rmax = -1; }
      }
    } else {
      for (int i = lane; i < p.Sq; i += 32) {
        const int lo = p.row_lo ? p.row_lo[(long long)b * p.Sq + i] : 0;
        const int hi = p.row_hi ? p.row_hi[(long long)b * p.Sq + i] : (p.causal ? i + 1 + shift : p.Sk);
        if (max(lo, kv0) < min(min(hi, p.Sk), kv0 + BKV)) { rmin = min(rmin, i); rmax = max(rmax, i); }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      rmin = min(rmin, __shfl_xor_sync(0xffffffffu, rmin, o));
      rmax = max(rmax, __shfl_xor_sync(0xffffffffu, rmax, o));
    }
    if (lane == 0) {
      q_range[0] = rmax >= 0 ? rmin / BQ : 0;
      q_range[1] = rmax >= 0 ? rmax / BQ + 1 : 0;
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int qb0 = q_range[0], qb1 = q_range[1];
  const int nblk = qb1 - qb0;
  const long long q_row_base = (long long)b * p.Sq;
  const long long k_row = (long long)b * p.Sk + kv0;

  if (warp == 0) {
    if (lane == 0 && nblk > 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmdO);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      tma_prefetch_desc(&tmdQ);
      constexpr int TILE_B = (HDIM / 64) * PANEL;   // bytes of a [128 x HDIM] tile
      mbar_expect_tx(kv_full, 2 * TILE_B);
      tma_load_2d(sK, &tmK, kv_full, hk * HDIM, (int)k_row);
      if (HDIM == 128) tma_load_2d(sK + PANEL, &tmK, kv_full, hk * HDIM + 64, (int)k_row);
      tma_load_2d(sV, &tmV, kv_full, hk * HDIM, (int)k_row);
      if (HDIM == 128) tma_load_2d(sV + PANEL, &tmV, kv_full, hk * HDIM + 64, (int)k_row);
      for (int it = 0; it < nblk; ++it) {
        const int qs = it & 1;
        const int qrow = (int)(q_row_base + (long long)(qb0 + it) * BQ);
        if (!mbar_wait(&q_free[qs], ((it >> 1) & 1) ^ 1, abort_flag, p.status)) break;
        mbar_expect_tx(&q_full[qs], TILE_B);
        tma_load_2d(sQ + qs * TILE, &tmQ, &q_full[qs], h * HDIM, qrow);
        if (HDIM == 128) tma_load_2d(sQ + qs * TILE + PANEL, &tmQ, &q_full[qs], h * HDIM + 64, qrow);
        if (!mbar_wait(do_free, (it & 1) ^ 1, abort_flag, p.status)) break;
        mbar_expect_tx(do_full, TILE_B);
        tma_load_2d(sdO, &tmdO, do_full, h * HDIM, qrow);
        if (HDIM == 128) tma_load_2d(sdO + PANEL, &tmdO, do_full, h * HDIM + 64, qrow);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && nblk > 0) {
      constexpr uint32_t id_kk = umma_idesc(128, 128, 1, 1, false, false);
      constexpr uint32_t id_mm = umma_idesc(128, HDIM, 1, 1, true, true);     // dV, dK: [keys x d]
      constexpr uint32_t id_km = umma_idesc(128, HDIM, 1, 1, false, true);    // dQ: [queries x d]
      const uint32_t adO = smem_u32(sdO), aK = smem_u32(sK), aV = smem_u32(sV), aP = smem_u32(sP), adS = smem_u32(sdS);
      const uint32_t tS = tmem_base, tdP = tmem_base + 128, tdV = tmem_base + 256, tdK = tmem_base + 384;
      // descriptors of every operand in the form(s) it is read in; the loops below only advance them
      // (scalars and selects: an array indexed at run time would live in local memory)
      const uint64_t dQk0 = umma_desc_sw128(smem_u32(sQ), 16, 1024), dQm0 = umma_desc_sw128(smem_u32(sQ), PANEL, 1024);
      const uint64_t dKk = umma_desc_sw128(aK, 16, 1024), dKm = umma_desc_sw128(aK, PANEL, 1024);
      const uint64_t dVk = umma_desc_sw128(aV, 16, 1024);
      const uint64_t dOk = umma_desc_sw128(adO, 16, 1024), dOm = umma_desc_sw128(adO, PANEL, 1024);
      const uint64_t dPm = umma_desc_sw128(aP, PANEL, 1024);
      const uint64_t dSk = umma_desc_sw128(adS, 16, 1024), dSm = umma_desc_sw128(adS, PANEL, 1024);
      auto issue_s = [&](int it) -> bool {   // S(it) = Q(it) K^T over d
        if (!mbar_wait(&q_full[it & 1], (it >> 1) & 1, abort_flag, p.status)) return false;
        tc_fence_after();
        const uint64_t qd = umma_desc_advance(dQk0, (it & 1) ? TILE : 0);
#pragma unroll
        for (int k = 0; k < HDIM / 16; ++k) {
          const uint32_t off = (k >> 2) * PANEL + (k & 3) * 32;
          umma_f16<1>(tS, umma_desc_advance(qd, off), umma_desc_advance(dKk, off), id_kk, k != 0);
        }
        umma_commit(s_full);
        return true;
      };
      auto issue_dp = [&](int it) -> bool {  // dP(it) = dO(it) V^T over d
        if (!mbar_wait(do_full, it & 1, abort_flag, p.status)) return false;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < HDIM / 16; ++k) {
          const uint32_t off = (k >> 2) * PANEL + (k & 3) * 32;
          umma_f16<1>(tdP, umma_desc_advance(dOk, off), umma_desc_advance(dVk, off), id_kk, k != 0);
        }
        umma_commit(dp_full);
        return true;
      };
      bool ok = mbar_wait(kv_full, 0, abort_flag, p.status);
      ok = ok && issue_s(0) && issue_dp(0);
      for (int it = 0; ok && it < nblk; ++it) {
        if (!mbar_wait(pds_full, it & 1, abort_flag, p.status)) break;
        tc_fence_after();
        if (it + 1 < nblk && !issue_s(it + 1)) break;
        const uint64_t qm = umma_desc_advance(dQm0, (it & 1) ? TILE : 0);
#pragma unroll
        for (int k = 0; k < 8; ++k)  // dV += P^T dO over q
          umma_f16<1>(tdV, umma_desc_advance(dPm, k * 2048), umma_desc_advance(dOm, k * 2048), id_mm, (it | k) != 0);
        umma_commit(do_free);
#pragma unroll
        for (int k = 0; k < 8; ++k)  // dK += dS^T Q over q
          umma_f16<1>(tdK, umma_desc_advance(dSm, k * 2048), umma_desc_advance(qm, k * 2048), id_mm, (it | k) != 0);
        umma_commit(&q_free[it & 1]);
        if constexpr (WITH_DQ) {
#pragma unroll
          for (int k = 0; k < 8; ++k) {  // dQ = dS K over keys (into the dP columns)
            const uint32_t off = (k >> 2) * PANEL + (k & 3) * 32;
            umma_f16<1>(tdP, umma_desc_advance(dSk, off), umma_desc_advance(dKm, k * 2048), id_km, k != 0);
          }
        }
        umma_commit(dq_full);
        if (it + 1 < nblk) {
          if constexpr (WITH_DQ) {
            if (!mbar_wait(dp_free, it & 1, abort_flag, p.status)) break;
            tc_fence_after();
          }
          if (!issue_dp(it + 1)) break;
        }
      }
    }
  } else {
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r = quarter * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const uint32_t tS = lane_addr + half * 64, tdP = lane_addr + 128 + half * 64;
    bool ok = true;

    auto row_info = [&](int it) -> RowInfo {
      RowInfo ri;
      ri.i = (qb0 + it) * BQ + r;
      ri.valid = it < nblk && ri.i < p.Sq;
      ri.lo = 0; ri.hi = 0; ri.lse2 = 0.f; ri.delta = 0.f;
      if (ri.valid) {
        const long long ridx = ((long long)b * p.Hq + h) * p.Sq + ri.i;
        const float l = p.lse[ridx];
        if (l == -INFINITY) {
          ri.valid = false;
        } else {
          ri.lse2 = l * 1.4426950408889634f;
          ri.delta = p.delta[ridx];
          ri.lo = p.row_lo ? p.row_lo[(long long)b * p.Sq + ri.i] : 0;
          ri.hi = p.row_hi ? p.row_hi[(long long)b * p.Sq + ri.i] : (p.causal ? ri.i + 1 + shift : p.Sk);
          ri.lo = max(ri.lo, 0);
          ri.hi = min(ri.hi, p.Sk);
        }
      }
      return ri;
    };
    // dQ(it) leaves the dP columns: registers -> staging tiles (four [128 x 32] fp32 boxes with the 128-byte
    // swizzle, in the memory of P and dS) -> reduce-add into the accumulation buffer by the TMA unit. Rows past
    // the end of the sequence hold zeros (their dS is zero), so whatever the tile covers there is unchanged.
    uint8_t* stage = sP;
    const bool reducer = threadIdx.x == 64;     // first element-wise thread issues the TMA operations
    auto drain_dq = [&](int it) -> bool {
      if (!__all_sync(0xffffffffu, mbar_wait(dq_full, it & 1, abort_flag, p.status))) return false;
      if constexpr (!WITH_DQ) return true;   // the products that read P and dS have completed: nothing to move
      tc_fence_after();
      // this thread's HDIM / 2 columns of dQ: boxes (2 half, 2 half + 1) for 128, box `half` for 64
      uint32_t t0[32], t1[32];
      const uint32_t dq_addr = lane_addr + 128 + half * (HDIM / 2);
      tmem_ld_32x32(dq_addr, t0);
      if (HDIM == 128) tmem_ld_32x32(dq_addr + 32, t1);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(dp_free);
      uint8_t* row0 = stage + (half * (HDIM / 64)) * 16384 + r * 128;
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) {
        const int slot = (ch ^ (r & 7)) << 4;
        *reinterpret_cast<uint4*>(row0 + slot) = make_uint4(t0[ch * 4], t0[ch * 4 + 1], t0[ch * 4 + 2], t0[ch * 4 + 3]);
        if (HDIM == 128)
          *reinterpret_cast<uint4*>(row0 + 16384 + slot) =
              make_uint4(t1[ch * 4], t1[ch * 4 + 1], t1[ch * 4 + 2], t1[ch * 4 + 3]);
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(stage_full);
      bool rok = true;
      if (reducer) {
        rok = mbar_wait(stage_full, it & 1, abort_flag, p.status);
        if (rok) {
          const int qrow = (int)(q_row_base + (long long)(qb0 + it) * BQ);
#pragma unroll
          for (int bx = 0; bx < HDIM / 32; ++bx)
            tma_reduce_add_2d(&tmdQ, stage + bx * 16384, h * HDIM + bx * 32, qrow);
          tma_store_commit();
          tma_store_wait_read<0>();
          mbar_arrive(stage_free);
        }
      }
      return __all_sync(0xffffffffu, rok);   // the whole warp leaves the loop together when a wait ran out
    };

    RowInfo cur = row_info(0);
    for (int it = 0; it < nblk; ++it) {
      const RowInfo nxt = row_info(it + 1);   // issued early: the loads complete under this block's work
      // warp-uniform, so that the per-element interval tests are a separate path that full tiles never enter
      const bool row_full = __all_sync(0xffffffffu, cur.valid && cur.lo <= kv0 && cur.hi >= kv0 + BKV);
      // ---- P(it) = exp2(S c - lse): runs while the tensor core accumulates dV, dK and forms dQ of block it-1
      if (!__all_sync(0xffffffffu, mbar_wait(s_full, it & 1, abort_flag, p.status))) { ok = false; break; }
      tc_fence_after();
      float pv[64];
      {
        uint32_t s0[32], s1[32];
        tmem_ld_32x32(tS, s0);
        tmem_ld_32x32(tS + 32, s1);
        tmem_ld_wait();
        const int c0 = kv0 + half * 64;
        if constexpr (BIAS) {
          if (cur.valid) {     // s + bias / scale, exactly as the forward pass formed it
            const __nv_bfloat16* bp = p.bias.ptr + (long long)b * p.bias.sb + (long long)h * p.bias.sh +
                                      (long long)cur.i * p.bias.sq + c0;
#pragma unroll
            for (int c8 = 0; c8 < 8; ++c8) {
              if (c0 + c8 * 8 < p.Sk) {
                const uint4 u = *reinterpret_cast<const uint4*>(bp + c8 * 8);
                const uint32_t w[4] = {u.x, u.y, u.z, u.w};
                uint32_t* d = (c8 < 4 ? s0 : s1) + (c8 & 3) * 8;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const float2 bv = unpack_bf16x2(w[j]);
                  d[2 * j] = __float_as_uint(fmaf(bv.x, p.inv_scale, __uint_as_float(d[2 * j])));
                  d[2 * j + 1] = __float_as_uint(fmaf(bv.y, p.inv_scale, __uint_as_float(d[2 * j + 1])));
                }
              }
            }
          }
        }
        const uint64_t sc2 = f2_pack(p.scale_log2, p.scale_log2), nl2 = f2_pack(-cur.lse2, -cur.lse2);
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
          float a0, a1, b0, b1;
          f2_unpack(f2_fma(f2_pack_bits(s0[c], s0[c + 1]), sc2, nl2), a0, a1);
          f2_unpack(f2_fma(f2_pack_bits(s1[c], s1[c + 1]), sc2, nl2), b0, b1);
          pv[c] = fast_exp2(a0); pv[c + 1] = fast_exp2(a1);
          pv[32 + c] = fast_exp2(b0); pv[33 + c] = fast_exp2(b1);
        }
        if (!row_full) {
#pragma unroll
          for (int c = 0; c < 64; ++c)
            if (!cur.valid || c0 + c < cur.lo || c0 + c >= cur.hi) pv[c] = 0.f;
        }
      }
      // ---- dQ(it-1) out of the dP columns, which frees them for dP(it)
      if (it > 0 && !drain_dq(it - 1)) { ok = false; break; }
      // ---- dS(it) = P (dP - delta) scale; P and dS to shared memory (free: dq_full(it-1) has been waited for)
      if (!__all_sync(0xffffffffu, mbar_wait(dp_full, it & 1, abort_flag, p.status))) { ok = false; break; }
      // P and dS share their memory with the staged dQ(it-1): wait until the TMA unit has read it
      if (WITH_DQ && it > 0 &&
          !__all_sync(0xffffffffu, mbar_wait(stage_free, (it - 1) & 1, abort_flag, p.status))) {
        ok = false;
        break;
      }
      tc_fence_after();
      uint8_t* prow = sP + half * PANEL + r * 128;
      uint8_t* dsrow = sdS + half * PANEL + r * 128;
      {
        uint32_t d0[32], d1[32];
        tmem_ld_32x32(tdP, d0);
        tmem_ld_32x32(tdP + 32, d1);
        tmem_ld_wait();
        const uint64_t nd2 = f2_pack(-cur.delta, -cur.delta), scl2 = f2_pack(p.scale, p.scale);
        if constexpr (!DROP) {
#pragma unroll
          for (int c8 = 0; c8 < 8; ++c8) {
            uint32_t pk[4], dk_[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const int c = c8 * 8 + 2 * q;
              const uint64_t dp2 = c < 32 ? f2_pack_bits(d0[c & 31], d0[(c + 1) & 31])
                                          : f2_pack_bits(d1[c & 31], d1[(c + 1) & 31]);
              const uint64_t p2 = f2_pack(pv[c], pv[c + 1]);
              float ds0, ds1;
              f2_unpack(f2_mul(f2_mul(p2, scl2), f2_add(dp2, nd2)), ds0, ds1);   // P (dP - delta) scale
              pk[q] = pack_bf16x2(pv[c], pv[c + 1]);
              dk_[q] = pack_bf16x2(ds0, ds1);
            }
            const int slot = (c8 ^ (r & 7)) << 4;
            *reinterpret_cast<uint4*>(prow + slot) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            *reinterpret_cast<uint4*>(dsrow + slot) = make_uint4(dk_[0], dk_[1], dk_[2], dk_[3]);
          }
        } else {
          // dropout: with m = keep / (1 - p) per element, the tile for dV is P m and dS = P (m dP - delta) scale
          const uint32_t dkey = drop_row_key(p.drop, (uint32_t)(b * p.Hq + h), (uint32_t)cur.i);
          const uint32_t cbase = (uint32_t)(kv0 + half * 64);
#pragma unroll
          for (int c8 = 0; c8 < 8; ++c8) {
            uint32_t pk[4], dk_[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const int c = c8 * 8 + 2 * q;
              const uint32_t w = drop_pair_bits(dkey, cbase + c);
              const float m0 = (w & 0xffffu) >= p.drop.thr16 ? p.drop.keep_scale : 0.f;
              const float m1 = (w >> 16) >= p.drop.thr16 ? p.drop.keep_scale : 0.f;
              const uint64_t m2 = f2_pack(m0, m1);
              const uint64_t dp2 = c < 32 ? f2_pack_bits(d0[c & 31], d0[(c + 1) & 31])
                                          : f2_pack_bits(d1[c & 31], d1[(c + 1) & 31]);
              const uint64_t p2 = f2_pack(pv[c], pv[c + 1]);
              float ds0, ds1, pm0, pm1;
              f2_unpack(f2_mul(f2_mul(p2, scl2), f2_fma(dp2, m2, nd2)), ds0, ds1);
              f2_unpack(f2_mul(p2, m2), pm0, pm1);
              pk[q] = pack_bf16x2(pm0, pm1);
              dk_[q] = pack_bf16x2(ds0, ds1);
            }
            const int slot = (c8 ^ (r & 7)) << 4;
            *reinterpret_cast<uint4*>(prow + slot) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            *reinterpret_cast<uint4*>(dsrow + slot) = make_uint4(dk_[0], dk_[1], dk_[2], dk_[3]);
          }
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(pds_full);
      cur = nxt;
    }
    if (ok && nblk > 0) ok = drain_dq(nblk - 1);
    if (WITH_DQ && reducer) tma_store_wait<0>();
    // dV / dK of this key block: TMEM lane = key row. tcgen05.ld is a warp-wide (.sync.aligned)
    // instruction: every lane executes it, only the global stores are predicated per row.
    const int j = kv0 + r;
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      const bool store = j < p.Sk;
      __nv_bfloat16* dvrow = p.dv + ((long long)b * p.Sk + j) * p.dkv_stride + h * HDIM + half * (HDIM / 2);
      __nv_bfloat16* dkrow = p.dk + ((long long)b * p.Sk + j) * p.dkv_stride + h * HDIM + half * (HDIM / 2);
      if (nblk > 0) tc_fence_after();
#pragma unroll
      for (int cc = 0; cc < HDIM / 64; ++cc) {
        uint32_t tv[32], tk[32];
        if (nblk > 0) {
          tmem_ld_32x32(lane_addr + 256 + half * (HDIM / 2) + cc * 32, tv);
          tmem_ld_32x32(lane_addr + 384 + half * (HDIM / 2) + cc * 32, tk);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int c = 0; c < 32; ++c) { tv[c] = 0u; tk[c] = 0u; }
        }
        if (store) {
#pragma unroll
          for (int c = 0; c < 32; c += 8) {
            uint4 a, d;
            a.x = pack_bf16x2(__uint_as_float(tv[c]), __uint_as_float(tv[c + 1]));
            a.y = pack_bf16x2(__uint_as_float(tv[c + 2]), __uint_as_float(tv[c + 3]));
            a.z = pack_bf16x2(__uint_as_float(tv[c + 4]), __uint_as_float(tv[c + 5]));
            a.w = pack_bf16x2(__uint_as_float(tv[c + 6]), __uint_as_float(tv[c + 7]));
            d.x = pack_bf16x2(__uint_as_float(tk[c]), __uint_as_float(tk[c + 1]));
            d.y = pack_bf16x2(__uint_as_float(tk[c + 2]), __uint_as_float(tk[c + 3]));
            d.z = pack_bf16x2(__uint_as_float(tk[c + 4]), __uint_as_float(tk[c + 5]));
            d.w = pack_bf16x2(__uint_as_float(tk[c + 6]), __uint_as_float(tk[c + 7]));
            *reinterpret_cast<uint4*>(dvrow + cc * 32 + c) = a;
            *reinterpret_cast<uint4*>(dkrow + cc * 32 + c) = d;
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    const uint64_t t_start = globaltimer_ns();
    while (globaltimer_ns() - t_start < 200000ull) __nanosleep(1000);
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<1>(tmem_base, 512);
  }
}

// delta[b, h, i] = sum_d dO[b, i, h, d] * O[b, i, h, d]; one warp per (b, i, h) row of hd (128 or 64) elements.
__global__ void flash_delta_kernel(const __nv_bfloat16* __restrict__ dO, const __nv_bfloat16* __restrict__ O,
                                   float* __restrict__ delta, int B, int Sq, int Hq, long long do_stride, int hd) {
  const long long w = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long total = (long long)B * Sq * Hq;
  if (w >= total) return;
  const int hh = (int)(w % Hq);
  const long long tok = w / Hq;  // b * Sq + i
  float s = 0.f;
  if (lane * 4 < hd) {
    const uint2 a = *reinterpret_cast<const uint2*>(dO + tok * do_stride + hh * hd + lane * 4);
    const uint2 o = *reinterpret_cast<const uint2*>(O + (tok * Hq + hh) * hd + lane * 4);
    const float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y), o0 = unpack_bf16x2(o.x), o1 = unpack_bf16x2(o.y);
    s = a0.x * o0.x + a0.y * o0.y + a1.x * o1.x + a1.y * o1.y;
  }
  s = warp_sum(s);
  if (lane == 0) {
    const long long bb = tok / Sq, i = tok % Sq;
    delta[(bb * Hq + hh) * Sq + i] = s;
  }
}

// src: [rows, row_elems] fp32 contiguous -> dst rows of pitch dst_stride (bf16)
__global__ void f32_to_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long long n4,
                                   int row_elems4, long long dst_stride) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    const float4 v = reinterpret_cast<const float4*>(src)[i];
    uint2 o;
    o.x = pack_bf16x2(v.x, v.y);
    o.y = pack_bf16x2(v.z, v.w);
    const long long row = i / row_elems4;
    const int c4 = (int)(i - row * row_elems4);
    *reinterpret_cast<uint2*>(dst + row * dst_stride + c4 * 4) = o;
  }
}

}  // namespace

extern "C" int atb_flash_bwd_dq(const void* dout, const void* q, const void* k, const void* v, const float* lse,
                                const float* delta, void* dq, const int* row_lo, const int* row_hi, int B, int Sq,
                                int Sk, int Hq, int Hkv, long long q_stride, long long k_stride, long long v_stride,
                                long long do_stride, long long dq_stride, int causal, float softmax_scale,
                                void* stream, int* status);

extern "C" int atb_flash_bwd_dkv(const void* dout, const void* q, const void* k, const void* v, const float* lse,
                                 const float* delta, void* dk, void* dv, const int* row_lo, const int* row_hi, int B,
                                 int Sq, int Sk, int Hq, int Hkv, long long q_stride, long long k_stride,
                                 long long v_stride, long long do_stride, long long dkv_stride, int causal,
                                 float softmax_scale, void* stream, int* status);

// Which key-block kernel the two-kernel form uses: 1 = flash_attn_bwd_dkv.cu (transposed products, P and dS kept
// in tensor memory), 0 = this file's kernel without its dQ part (P and dS through shared memory), -1 (default) =
// by shape: measured at H=32, D=128 the shared-memory form is ahead up to 4096 keys (667 vs 681 us causal, 1067
// vs 1281 us full) and the transposed form from 8192 causal keys on (2121 vs 2151 us).
static int g_dkv_transposed = -1;
extern "C" void atb_flash_bwd_set_dkv(int transposed) { g_dkv_transposed = transposed; }

// Two forms. dq_acc == nullptr (default of the Python wrapper): the key-block kernel writes dK and dV, the
// query-block kernel of flash_attn_bwd_dq.cu writes dQ; no atomics, results do not depend on scheduling.
// dq_acc != nullptr: one key-block kernel for all three; dQ goes through TMA reduce-adds into dq_acc
// (fp32 [B, Sq, Hq, 128], zero on entry) and a conversion pass.
// dq_acc must be zero on entry; dq/dk/dv are written as token-major rows of pitch dq_stride / dkv_stride
// elements (so they may be slices of one fused [tokens, (Hq + 2 Hq) * 128] gradient buffer). dk, dv are per
// query head; the caller sums head groups for grouped-query attention. `delta` is scratch [B, Hq, Sq].
// One-kernel form (dQ through the fp32 buffer) for a given dropout / bias / head-dim combination.
template <bool DROP, bool BIAS, int HDIM>
static int bwd_variant(dim3 grid, cudaStream_t st, const CUtensorMap& tmQ, const CUtensorMap& tmdO, const CUtensorMap& tmK,
                       const CUtensorMap& tmV, const CUtensorMap& tmdQ, const BwdParams& p) {
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(flash_bwd_kernel<true, DROP, BIAS, HDIM>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             SmemB::TOTAL) != cudaSuccess)
      return -4;
    attr_set = true;
  }
  flash_bwd_kernel<true, DROP, BIAS, HDIM><<<grid, THREADS, SmemB::TOTAL, st>>>(tmQ, tmdO, tmK, tmV, tmdQ, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

static int flash_bwd_launch(const void* dout, const void* q, const void* k, const void* v, const void* out,
                            const float* lse, float* delta, float* dq_acc, void* dq, void* dk, void* dv,
                            const int* row_lo, const int* row_hi, int B, int Sq, int Sk, int Hq, int Hkv,
                            long long q_stride, long long k_stride, long long v_stride, long long do_stride,
                            long long dq_stride, long long dkv_stride, int causal, float softmax_scale, void* stream,
                            int* status, DropParams drop, BiasParams bias = BiasParams{nullptr, 0, 0, 0},
                            int head_dim = 128) {
  if (B <= 0 || Sq <= 0 || Sk <= 0) return 0;
  // dropout, the additive bias and head dim 64 are implemented in the one-kernel form only
  if (head_dim != 128 && head_dim != 64) return -1;
  const int HDv = head_dim;
  if ((drop.thr16 != 0 || bias.ptr != nullptr || HDv != 128) && dq_acc == nullptr) return -1;
  if (bias.ptr != nullptr &&
      ((Sk & 7) || ((bias.sb | bias.sh | bias.sq) & 7) || (reinterpret_cast<uintptr_t>(bias.ptr) & 15) ||
       !(softmax_scale > 0.f)))
    return -1;
  if (Hq % Hkv) return -1;
  if ((q_stride | k_stride | v_stride | do_stride | dq_stride | dkv_stride) & 7) return -1;
  cudaStream_t st = (cudaStream_t)stream;
  CUtensorMap tmQ, tmdO, tmK, tmV, tmdQ;
  if (!make_tmap_2d(&tmQ, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)B * Sq, (uint64_t)Hq * HDv, q_stride, BQ, 64,
                    CU_TENSOR_MAP_SWIZZLE_128B))
    return -2;
  if (!make_tmap_2d(&tmdO, dout, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)B * Sq, (uint64_t)Hq * HDv, do_stride,
                    BQ, 64, CU_TENSOR_MAP_SWIZZLE_128B))
    return -2;
  if (!make_tmap_2d(&tmK, k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)B * Sk, (uint64_t)Hkv * HDv, k_stride, BKV,
                    64, CU_TENSOR_MAP_SWIZZLE_128B))
    return -2;
  if (!make_tmap_2d(&tmV, v, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)B * Sk, (uint64_t)Hkv * HDv, v_stride, BKV,
                    64, CU_TENSOR_MAP_SWIZZLE_128B))
    return -2;
  // fp32 accumulation buffer as [B*Sq, Hq*HD]; the kernel adds [128 x 32] boxes to it
  if (dq_acc == nullptr) {
    tmdQ = tmQ;   // unused by the kernel variant without dQ
  } else if (!make_tmap_2d(&tmdQ, dq_acc, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (uint64_t)B * Sq, (uint64_t)Hq * HDv,
                           (uint64_t)Hq * HDv, BQ, 32, CU_TENSOR_MAP_SWIZZLE_128B)) {
    return -2;
  }
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(flash_bwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SmemB::TOTAL) !=
        cudaSuccess)
      return -4;
    attr_set = true;
  }
  {
    const long long warps = (long long)B * Sq * Hq;
    const int threads = 256;
    const long long blocks = (warps * 32 + threads - 1) / threads;
    flash_delta_kernel<<<(unsigned)blocks, threads, 0, st>>>((const __nv_bfloat16*)dout, (const __nv_bfloat16*)out,
                                                             delta, B, Sq, Hq, do_stride, HDv);
  }
  BwdParams p;
  p.lse = lse; p.delta = delta; p.dq_acc = dq_acc; p.dk = (__nv_bfloat16*)dk; p.dv = (__nv_bfloat16*)dv;
  p.dkv_stride = dkv_stride;
  p.row_lo = row_lo; p.row_hi = row_hi;
  p.B = B; p.Sq = Sq; p.Sk = Sk; p.Hq = Hq; p.Hkv = Hkv; p.causal = causal;
  p.scale = softmax_scale; p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.status = status;
  p.drop = drop;
  p.bias = bias;
  p.inv_scale = 1.f / softmax_scale;
  dim3 grid((Sk + BKV - 1) / BKV, Hq, B);
  if (dq_acc == nullptr) {
    if (g_dkv_transposed > 0 || (g_dkv_transposed < 0 && causal && Sk >= 8192)) {
      const int rc = atb_flash_bwd_dkv(dout, q, k, v, lse, delta, dk, dv, row_lo, row_hi, B, Sq, Sk, Hq, Hkv, q_stride,
                                       k_stride, v_stride, do_stride, dkv_stride, causal, softmax_scale, stream, status);
      if (rc != 0) return rc;
    } else {
      flash_bwd_kernel<false><<<grid, THREADS, SmemB::TOTAL, st>>>(tmQ, tmdO, tmK, tmV, tmdQ, p);
      if (cudaGetLastError() != cudaSuccess) return -5;
    }
    return atb_flash_bwd_dq(dout, q, k, v, lse, delta, dq, row_lo, row_hi, B, Sq, Sk, Hq, Hkv, q_stride, k_stride,
                            v_stride, do_stride, dq_stride, causal, softmax_scale, stream, status);
  }
  {
    const bool dr = drop.thr16 != 0, bi = bias.ptr != nullptr;
    int rc;
#define ATB_BWD_PICK(HD_)                                                                          \
  rc = (dr && bi) ? bwd_variant<true, true, HD_>(grid, st, tmQ, tmdO, tmK, tmV, tmdQ, p)            \
       : dr       ? bwd_variant<true, false, HD_>(grid, st, tmQ, tmdO, tmK, tmV, tmdQ, p)           \
       : bi       ? bwd_variant<false, true, HD_>(grid, st, tmQ, tmdO, tmK, tmV, tmdQ, p)           \
                  : bwd_variant<false, false, HD_>(grid, st, tmQ, tmdO, tmK, tmV, tmdQ, p)
    if (HDv == 64) ATB_BWD_PICK(64); else ATB_BWD_PICK(128);
#undef ATB_BWD_PICK
    if (rc != 0) return rc;
  }
  const long long n4 = (long long)B * Sq * Hq * HDv / 4;
  long long g = (n4 + 255) / 256;
  if (g > 148 * 16) g = 148 * 16;
  f32_to_bf16_kernel<<<(unsigned)g, 256, 0, st>>>(dq_acc, (__nv_bfloat16*)dq, n4, Hq * HDv / 4, dq_stride);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

extern "C" int atb_flash_bwd(const void* dout, const void* q, const void* k, const void* v, const void* out,
                             const float* lse, float* delta, float* dq_acc, void* dq, void* dk, void* dv,
                             const int* row_lo, const int* row_hi, int B, int Sq, int Sk, int Hq, int Hkv,
                             long long q_stride, long long k_stride, long long v_stride, long long do_stride,
                             long long dq_stride, long long dkv_stride, int causal, float softmax_scale, void* stream,
                             int* status) {
  return flash_bwd_launch(dout, q, k, v, out, lse, delta, dq_acc, dq, dk, dv, row_lo, row_hi, B, Sq, Sk, Hq, Hkv,
                          q_stride, k_stride, v_stride, do_stride, dq_stride, dkv_stride, causal, softmax_scale, stream,
                          status, DropParams{0u, 0u, 0u, 1.f});
}

// Backward of atb_flash_fwd_dropout: same thr16 and seed pair as the forward; one-kernel form (dq_acc required).
extern "C" int atb_flash_bwd_dropout(const void* dout, const void* q, const void* k, const void* v, const void* out,
                                     const float* lse, float* delta, float* dq_acc, void* dq, void* dk, void* dv,
                                     const int* row_lo, const int* row_hi, int B, int Sq, int Sk, int Hq, int Hkv,
                                     long long q_stride, long long k_stride, long long v_stride, long long do_stride,
                                     long long dq_stride, long long dkv_stride, int causal, float softmax_scale,
                                     void* stream, int* status, unsigned thr16, unsigned seed_lo, unsigned seed_hi) {
  if (thr16 == 0 || thr16 >= 65536u) return -1;
  return flash_bwd_launch(dout, q, k, v, out, lse, delta, dq_acc, dq, dk, dv, row_lo, row_hi, B, Sq, Sk, Hq, Hkv,
                          q_stride, k_stride, v_stride, do_stride, dq_stride, dkv_stride, causal, softmax_scale, stream,
                          status, DropParams{thr16, seed_lo, seed_hi, 65536.f / (float)(65536u - thr16)});
}

// Backward of atb_flash_fwd_bias: the same bias (it gets no gradient) and, if thr16 != 0, the same dropout.
extern "C" int atb_flash_bwd_bias(const void* dout, const void* q, const void* k, const void* v, const void* out,
                                  const float* lse, float* delta, float* dq_acc, void* dq, void* dk, void* dv,
                                  const int* row_lo, const int* row_hi, int B, int Sq, int Sk, int Hq, int Hkv,
                                  long long q_stride, long long k_stride, long long v_stride, long long do_stride,
                                  long long dq_stride, long long dkv_stride, int causal, float softmax_scale,
                                  void* stream, int* status, unsigned thr16, unsigned seed_lo, unsigned seed_hi,
                                  const void* bias, long long bias_sb, long long bias_sh, long long bias_sq) {
  if (thr16 >= 65536u || bias == nullptr) return -1;
  const DropParams drop = thr16 ? DropParams{thr16, seed_lo, seed_hi, 65536.f / (float)(65536u - thr16)}
                                : DropParams{0u, 0u, 0u, 1.f};
  return flash_bwd_launch(dout, q, k, v, out, lse, delta, dq_acc, dq, dk, dv, row_lo, row_hi, B, Sq, Sk, Hq, Hkv,
                          q_stride, k_stride, v_stride, do_stride, dq_stride, dkv_stride, causal, softmax_scale, stream,
                          status, drop, BiasParams{(const __nv_bfloat16*)bias, bias_sb, bias_sh, bias_sq});
}

// The general entry point: head dim 128 or 64, optional dropout (thr16 != 0) and additive bias (bias != null).
// Anything but the plain head-dim-128 case needs dq_acc (one-kernel form).
extern "C" int atb_flash_bwd_ex(const void* dout, const void* q, const void* k, const void* v, const void* out,
                                const float* lse, float* delta, float* dq_acc, void* dq, void* dk, void* dv,
                                const int* row_lo, const int* row_hi, int B, int Sq, int Sk, int Hq, int Hkv,
                                long long q_stride, long long k_stride, long long v_stride, long long do_stride,
                                long long dq_stride, long long dkv_stride, int causal, float softmax_scale,
                                void* stream, int* status, unsigned thr16, unsigned seed_lo, unsigned seed_hi,
                                const void* bias, long long bias_sb, long long bias_sh, long long bias_sq,
                                int head_dim) {
  if (thr16 >= 65536u) return -1;
  const DropParams drop = thr16 ? DropParams{thr16, seed_lo, seed_hi, 65536.f / (float)(65536u - thr16)}
                                : DropParams{0u, 0u, 0u, 1.f};
  return flash_bwd_launch(dout, q, k, v, out, lse, delta, dq_acc, dq, dk, dv, row_lo, row_hi, B, Sq, Sk, Hq, Hkv,
                          q_stride, k_stride, v_stride, do_stride, dq_stride, dkv_stride, causal, softmax_scale, stream,
                          status, drop, BiasParams{(const __nv_bfloat16*)bias, bias_sb, bias_sh, bias_sq}, head_dim);
}
