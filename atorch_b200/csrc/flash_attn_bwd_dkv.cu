// Flash attention backward, key/value-gradient kernel for sm_100a (head dim 128, bf16), tcgen05 + TMEM + TMA.
//
// One CTA per (128 keys, head, batch) walks the query blocks that can see its keys and accumulates dV and dK in
// tensor memory. Everything is computed transposed, so that the element-wise results are already what the next
// products want as their tensor-memory operand and never touch shared memory:
//   S^T  = K Q^T,  dP^T = V dO^T                    smem x smem -> TMEM   (lane = key, column = query)
//   P^T  = exp2(S^T c - lse[q]),  dS^T = P^T (dP^T - delta[q]) s     registers; bf16 written over S^T / dP^T
//   dV  += P^T dO,  dK += dS^T Q                     TMEM x smem (MN-major dO, Q) -> TMEM
// TMEM: S^T | dP^T | dV | dK = 4 x 128 columns. With P and dS out of shared memory, Q and dO are both
// double-buffered (K, V: 64 KB once; Q, dO: 128 KB), the per-query values lse, delta and the key interval of the
// next block are staged in 2 KB of shared memory by the producer warp, and the tensor core alternates
//   [dV(i), S^T(i+1)]  while the warps form dS^T(i)   and   [dK(i), dP^T(i+1)]  while they form P^T(i+1).
// The query gradient comes from flash_attn_bwd_dq.cu.
//
// Warp 0 = producer (TMA loads by lane 0, row values by all lanes), warp 1 = MMA issuer / TMEM owner, warps 2..9 =
// element-wise work: thread (key row r, half h) owns query columns [64h, 64h+64). The bf16 results of one half
// overwrite fp32 columns the other half reads, so the two warps of a lane quarter meet at a bounded barrier
// between loading and storing. Masks are per-query key intervals [lo, hi) as in the forward kernel.
#include "common.cuh"

namespace {
using namespace atb;

constexpr int BQ = 128, BKV = 128, HD = 128;
constexpr int PANEL = 128 * 64 * 2;
constexpr int TILE = 2 * PANEL;
constexpr int N_EW = 256;
constexpr int THREADS = 64 + N_EW;

struct DkvParams {
  const float* lse;    // [B, Hq, Sq]
  const float* delta;  // [B, Hq, Sq]
  __nv_bfloat16* dk;   // token-major, head h at columns [h*HD, h*HD+HD) of a row of pitch dkv_stride
  __nv_bfloat16* dv;
  long long dkv_stride;
  const int* row_lo;
  const int* row_hi;
  int B, Sq, Sk, Hq, Hkv, causal;
  float scale, scale_log2;
  int* status;
};

struct RowVals {          // per query row of a block, as the element-wise threads want them
  float neg_lse2[BQ];     // -lse * log2(e); -inf for rows that take no part (P becomes 0)
  float neg_delta[BQ];
  int lo[BQ], hi[BQ];
};

struct SmemK {
  static constexpr int K_OFF = 0;
  static constexpr int V_OFF = K_OFF + TILE;
  static constexpr int Q_OFF = V_OFF + TILE;          // two stages
  static constexpr int DO_OFF = Q_OFF + 2 * TILE;     // two stages
  static constexpr int ROWS_OFF = DO_OFF + 2 * TILE;  // 192 KB; two RowVals
  static constexpr int BAR_OFF = ROWS_OFF + 2 * (int)sizeof(RowVals);
  static constexpr int NBARS = 1 + 4 + 4 + 2 + 2 + 2 + 1 + 8;
  static constexpr int TOTAL = BAR_OFF + NBARS * 8 + 64 + 1024;
};
static_assert(SmemK::TOTAL <= 232448, "shared memory of the dK/dV kernel exceeds 227 KB");

__global__ void __launch_bounds__(THREADS, 1)
flash_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmdO,
                     const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, DkvParams p) {
  using L = SmemK;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem + L::K_OFF;
  uint8_t* sV = smem + L::V_OFF;
  uint8_t* sQ = smem + L::Q_OFF;
  uint8_t* sdO = smem + L::DO_OFF;
  RowVals* rows = reinterpret_cast<RowVals*>(smem + L::ROWS_OFF);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* kv_full = bars;
  uint64_t* q_full = bars + 1;     // [2]
  uint64_t* q_free = bars + 3;     // [2]  dK(i) has read Q(i); also frees the row values of that stage
  uint64_t* do_full = bars + 5;    // [2]
  uint64_t* do_free = bars + 7;    // [2]  dV(i) has read dO(i)
  uint64_t* rows_full = bars + 9;  // [2]
  uint64_t* st_full = bars + 11;   // S^T(i) is in TMEM
  uint64_t* dpt_full = bars + 12;  // dP^T(i) is in TMEM
  uint64_t* p_full = bars + 13;    // P^T(i) is in TMEM (all element-wise warps)
  uint64_t* ds_full = bars + 14;   // dS^T(i) is in TMEM
  uint64_t* acc_full = bars + 15;  // the last accumulating product has completed
  uint64_t* pair_a = bars + 16;    // [4] both warps of a lane quarter hold S^T(i)
  uint64_t* pair_c = bars + 20;    // [4] ... hold dP^T(i)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + L::NBARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* q_range = const_cast<int*>(reinterpret_cast<volatile int*>(tmem_slot + 2));  // [2]: first, last+1 q block

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != 0) return;
  const int kb = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.Hq / p.Hkv);
  const int kv0 = kb * BKV;
  const int shift = p.Sk - p.Sq;
  const bool analytic = p.row_lo == nullptr && p.row_hi == nullptr;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1); mbar_init(&q_free[i], 1);
      mbar_init(&do_full[i], 1); mbar_init(&do_free[i], 1);
      mbar_init(&rows_full[i], 1);
    }
    mbar_init(st_full, 1);
    mbar_init(dpt_full, 1);
    mbar_init(p_full, N_EW / 32);
    mbar_init(ds_full, N_EW / 32);
    mbar_init(acc_full, 1);
    for (int i = 0; i < 4; ++i) { mbar_init(&pair_a[i], 2); mbar_init(&pair_c[i], 2); }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc<1>(tmem_slot, 512);
    tmem_relinquish<1>();
  }
  if (warp == 2) {   // query rows whose interval meets this key block
    int rmin = INT_MAX, rmax = -1;
    if (analytic) {
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
  const int qb0 = q_range[0], nblk = q_range[1] - q_range[0];
  const long long q_row_base = (long long)b * p.Sq;
  const long long k_row = (long long)b * p.Sk + kv0;
  const uint32_t tSt = tmem_base, tdPt = tmem_base + 128, tdV = tmem_base + 256, tdK = tmem_base + 384;

  if (warp == 0) {
    if (nblk > 0) {
      if (lane == 0) {
        tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmdO); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
        mbar_expect_tx(kv_full, 2 * TILE);
        tma_load_2d(sK, &tmK, kv_full, hk * HD, (int)k_row);
        tma_load_2d(sK + PANEL, &tmK, kv_full, hk * HD + 64, (int)k_row);
        tma_load_2d(sV, &tmV, kv_full, hk * HD, (int)k_row);
        tma_load_2d(sV + PANEL, &tmV, kv_full, hk * HD + 64, (int)k_row);
      }
      for (int it = 0; it < nblk; ++it) {
        const int st = it & 1;
        const uint32_t ph = ((it >> 1) & 1) ^ 1;
        const int qrow = (int)(q_row_base + (long long)(qb0 + it) * BQ);
        bool ok = true;
        if (lane == 0) {
          ok = mbar_wait(&q_free[st], ph, abort_flag, p.status);
          if (ok) {
            mbar_expect_tx(&q_full[st], TILE);
            tma_load_2d(sQ + st * TILE, &tmQ, &q_full[st], h * HD, qrow);
            tma_load_2d(sQ + st * TILE + PANEL, &tmQ, &q_full[st], h * HD + 64, qrow);
          }
        }
        if (!__shfl_sync(0xffffffffu, (int)ok, 0)) break;
        // row values of this query block (the stage is free: q_free covers its previous user)
        RowVals& rv = rows[st];
#pragma unroll
        for (int e = 0; e < BQ / 32; ++e) {
          const int r = lane + 32 * e;
          const int i = (qb0 + it) * BQ + r;
          float nl = -INFINITY, nd = 0.f;
          int lo = 0, hi = 0;
          if (i < p.Sq) {
            const long long ridx = ((long long)b * p.Hq + h) * p.Sq + i;
            const float l = p.lse[ridx];
            if (l != -INFINITY) {
              nl = -l * 1.4426950408889634f;
              nd = -p.delta[ridx];
              lo = p.row_lo ? p.row_lo[(long long)b * p.Sq + i] : 0;
              hi = p.row_hi ? p.row_hi[(long long)b * p.Sq + i] : (p.causal ? i + 1 + shift : p.Sk);
              lo = max(lo, 0);
              hi = min(hi, p.Sk);
            }
          }
          rv.neg_lse2[r] = nl; rv.neg_delta[r] = nd; rv.lo[r] = lo; rv.hi[r] = hi;
        }
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&rows_full[st]);
          ok = mbar_wait(&do_free[st], ph, abort_flag, p.status);
          if (ok) {
            mbar_expect_tx(&do_full[st], TILE);
            tma_load_2d(sdO + st * TILE, &tmdO, &do_full[st], h * HD, qrow);
            tma_load_2d(sdO + st * TILE + PANEL, &tmdO, &do_full[st], h * HD + 64, qrow);
          }
        }
        if (!__shfl_sync(0xffffffffu, (int)ok, 0)) break;
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && nblk > 0) {
      constexpr uint32_t id_kk = umma_idesc(128, 128, 1, 1, false, false);
      constexpr uint32_t id_km = umma_idesc(128, 128, 1, 1, false, true);
      const uint64_t dKk = umma_desc_sw128(smem_u32(sK), 16, 1024), dVk = umma_desc_sw128(smem_u32(sV), 16, 1024);
      const uint64_t dQk0 = umma_desc_sw128(smem_u32(sQ), 16, 1024), dQm0 = umma_desc_sw128(smem_u32(sQ), PANEL, 1024);
      const uint64_t dOk0 = umma_desc_sw128(smem_u32(sdO), 16, 1024), dOm0 = umma_desc_sw128(smem_u32(sdO), PANEL, 1024);
      auto issue_st = [&](int it) -> bool {   // S^T(it) = K Q(it)^T
        if (!mbar_wait(&q_full[it & 1], (it >> 1) & 1, abort_flag, p.status)) return false;
        tc_fence_after();
        const uint64_t qd = umma_desc_advance(dQk0, (it & 1) ? TILE : 0);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t off = (k >> 2) * PANEL + (k & 3) * 32;
          umma_f16<1>(tSt, umma_desc_advance(dKk, off), umma_desc_advance(qd, off), id_kk, k != 0);
        }
        umma_commit(st_full);
        return true;
      };
      auto issue_dpt = [&](int it) -> bool {  // dP^T(it) = V dO(it)^T
        if (!mbar_wait(&do_full[it & 1], (it >> 1) & 1, abort_flag, p.status)) return false;
        tc_fence_after();
        const uint64_t od = umma_desc_advance(dOk0, (it & 1) ? TILE : 0);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t off = (k >> 2) * PANEL + (k & 3) * 32;
          umma_f16<1>(tdPt, umma_desc_advance(dVk, off), umma_desc_advance(od, off), id_kk, k != 0);
        }
        umma_commit(dpt_full);
        return true;
      };
      bool ok = mbar_wait(kv_full, 0, abort_flag, p.status);
      ok = ok && issue_st(0) && issue_dpt(0);
      for (int it = 0; ok && it < nblk; ++it) {
        const int st = it & 1;
        if (!mbar_wait(p_full, it & 1, abort_flag, p.status)) break;
        tc_fence_after();
        const uint64_t om = umma_desc_advance(dOm0, st ? TILE : 0);
#pragma unroll
        for (int k = 0; k < 8; ++k)   // dV += P^T dO(it): 16 queries per step = 8 TMEM columns of packed bf16
          umma_f16_ts(tdV, tSt + k * 8, umma_desc_advance(om, k * 2048), id_km, (it | k) != 0);
        umma_commit(&do_free[st]);
        if (it + 1 < nblk && !issue_st(it + 1)) break;
        if (!mbar_wait(ds_full, it & 1, abort_flag, p.status)) break;
        tc_fence_after();
        const uint64_t qm = umma_desc_advance(dQm0, st ? TILE : 0);
#pragma unroll
        for (int k = 0; k < 8; ++k)   // dK += dS^T Q(it)
          umma_f16_ts(tdK, tdPt + k * 8, umma_desc_advance(qm, k * 2048), id_km, (it | k) != 0);
        umma_commit(&q_free[st]);
        if (it + 1 < nblk && !issue_dpt(it + 1)) break;
        if (it == nblk - 1) umma_commit(acc_full);
      }
    }
  } else {
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r = quarter * 32 + lane;
    const int kk = kv0 + r;                       // this thread's key
    const uint32_t lane_addr = ((uint32_t)(quarter * 32) << 16);
    const uint64_t sc2 = f2_pack(p.scale_log2, p.scale_log2), scl2 = f2_pack(p.scale, p.scale);
    bool ok = true;
    for (int it = 0; it < nblk; ++it) {
      const RowVals& rv = rows[it & 1];
      const int i0 = (qb0 + it) * BQ;             // first query row of the block
      // every query of the block sees every key of this block: no per-element tests (warp-uniform)
      const bool full = analytic && (!p.causal || i0 + shift + 1 >= kv0 + BKV) && (kv0 + BKV <= p.Sk);
      if (!__all_sync(0xffffffffu, mbar_wait(&rows_full[it & 1], (it >> 1) & 1, abort_flag, p.status))) { ok = false; break; }
      // ---- P^T(it) = exp2(S^T c - lse[q])
      if (!__all_sync(0xffffffffu, mbar_wait(st_full, it & 1, abort_flag, p.status))) { ok = false; break; }
      tc_fence_after();
      float pv[64];
      {
        uint32_t s0[32], s1[32];
        tmem_ld_32x32(tSt + lane_addr + half * 64, s0);
        tmem_ld_32x32(tSt + lane_addr + half * 64 + 32, s1);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&pair_a[quarter]);
        const float2* nl = reinterpret_cast<const float2*>(rv.neg_lse2 + half * 64);
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
          const float2 la = nl[c >> 1], lb = nl[16 + (c >> 1)];
          float a0, a1, b0, b1;
          f2_unpack(f2_fma(f2_pack_bits(s0[c], s0[c + 1]), sc2, f2_pack(la.x, la.y)), a0, a1);
          f2_unpack(f2_fma(f2_pack_bits(s1[c], s1[c + 1]), sc2, f2_pack(lb.x, lb.y)), b0, b1);
          pv[c] = fast_exp2(a0); pv[c + 1] = fast_exp2(a1);
          pv[32 + c] = fast_exp2(b0); pv[33 + c] = fast_exp2(b1);
        }
        if (!full) {
          const int* lo = rv.lo + half * 64;
          const int* hi = rv.hi + half * 64;
#pragma unroll
          for (int c = 0; c < 64; ++c)
            if (kk < lo[c] || kk >= hi[c]) pv[c] = 0.f;
        }
        uint32_t pk[32];
#pragma unroll
        for (int c = 0; c < 64; c += 2) pk[c >> 1] = pack_bf16x2(pv[c], pv[c + 1]);
        // the other half's thread of this key row must hold its S^T before these columns are overwritten
        if (!__all_sync(0xffffffffu, mbar_wait(&pair_a[quarter], it & 1, abort_flag, p.status))) { ok = false; break; }
        tmem_st_32x32(tSt + lane_addr + half * 32, pk);   // queries [64h, 64h+64) as packed bf16: columns [32h, 32h+32)
        tmem_st_wait();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
      // ---- dS^T(it) = P^T (dP^T - delta[q]) scale
      if (!__all_sync(0xffffffffu, mbar_wait(dpt_full, it & 1, abort_flag, p.status))) { ok = false; break; }
      tc_fence_after();
      {
        uint32_t d0[32], d1[32];
        tmem_ld_32x32(tdPt + lane_addr + half * 64, d0);
        tmem_ld_32x32(tdPt + lane_addr + half * 64 + 32, d1);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&pair_c[quarter]);
        const float2* nd = reinterpret_cast<const float2*>(rv.neg_delta + half * 64);
        uint32_t dk_[32];
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
          const float2 da = nd[c >> 1], db = nd[16 + (c >> 1)];
          float x0, x1, y0, y1;
          f2_unpack(f2_mul(f2_mul(f2_pack(pv[c], pv[c + 1]), scl2),
                           f2_add(f2_pack_bits(d0[c], d0[c + 1]), f2_pack(da.x, da.y))), x0, x1);
          f2_unpack(f2_mul(f2_mul(f2_pack(pv[32 + c], pv[33 + c]), scl2),
                           f2_add(f2_pack_bits(d1[c], d1[c + 1]), f2_pack(db.x, db.y))), y0, y1);
          dk_[c >> 1] = pack_bf16x2(x0, x1);
          dk_[16 + (c >> 1)] = pack_bf16x2(y0, y1);
        }
        if (!__all_sync(0xffffffffu, mbar_wait(&pair_c[quarter], it & 1, abort_flag, p.status))) { ok = false; break; }
        tmem_st_32x32(tdPt + lane_addr + half * 32, dk_);
        tmem_st_wait();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_full);
    }
    // dV / dK of this key block: TMEM lane = key row. tcgen05.ld is a warp-wide (.sync.aligned) instruction:
    // every lane executes it, only the global stores are predicated per row.
    ok = __all_sync(0xffffffffu, ok);
    if (ok && nblk > 0) ok = __all_sync(0xffffffffu, mbar_wait(acc_full, 0, abort_flag, p.status));
    if (ok) {
      const bool store = kk < p.Sk;
      __nv_bfloat16* dvrow = p.dv + ((long long)b * p.Sk + kk) * p.dkv_stride + h * HD + half * 64;
      __nv_bfloat16* dkrow = p.dk + ((long long)b * p.Sk + kk) * p.dkv_stride + h * HD + half * 64;
      if (nblk > 0) tc_fence_after();
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        uint32_t tv[32], tk[32];
        if (nblk > 0) {
          tmem_ld_32x32(tdV + lane_addr + half * 64 + cc * 32, tv);
          tmem_ld_32x32(tdK + lane_addr + half * 64 + cc * 32, tk);
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

}  // namespace

// dk, dv: token-major rows of pitch dkv_stride elements, per query head (the caller sums head groups for
// grouped-query attention); lse, delta: [B, Hq, Sq] fp32.
extern "C" int atb_flash_bwd_dkv(const void* dout, const void* q, const void* k, const void* v, const float* lse,
                                 const float* delta, void* dk, void* dv, const int* row_lo, const int* row_hi, int B,
                                 int Sq, int Sk, int Hq, int Hkv, long long q_stride, long long k_stride,
                                 long long v_stride, long long do_stride, long long dkv_stride, int causal,
                                 float softmax_scale, void* stream, int* status) {
  if (B <= 0 || Sq <= 0 || Sk <= 0) return 0;
  if (Hq % Hkv) return -1;
  if ((q_stride | k_stride | v_stride | do_stride | dkv_stride) & 7) return -1;
  CUtensorMap tmQ, tmdO, tmK, tmV;
  if (!make_tmap_2d(&tmQ, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)B * Sq, (uint64_t)Hq * HD, q_stride, BQ, 64,
                    CU_TENSOR_MAP_SWIZZLE_128B))
    return -2;
  if (!make_tmap_2d(&tmdO, dout, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)B * Sq, (uint64_t)Hq * HD, do_stride,
                    BQ, 64, CU_TENSOR_MAP_SWIZZLE_128B))
    return -2;
  if (!make_tmap_2d(&tmK, k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)B * Sk, (uint64_t)Hkv * HD, k_stride, BKV,
                    64, CU_TENSOR_MAP_SWIZZLE_128B))
    return -2;
  if (!make_tmap_2d(&tmV, v, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)B * Sk, (uint64_t)Hkv * HD, v_stride, BKV,
                    64, CU_TENSOR_MAP_SWIZZLE_128B))
    return -2;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(flash_bwd_dkv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SmemK::TOTAL) !=
        cudaSuccess)
      return -4;
    attr_set = true;
  }
  DkvParams p;
  p.lse = lse; p.delta = delta; p.dk = (__nv_bfloat16*)dk; p.dv = (__nv_bfloat16*)dv; p.dkv_stride = dkv_stride;
  p.row_lo = row_lo; p.row_hi = row_hi;
  p.B = B; p.Sq = Sq; p.Sk = Sk; p.Hq = Hq; p.Hkv = Hkv; p.causal = causal;
  p.scale = softmax_scale; p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.status = status;
  dim3 grid((Sk + BKV - 1) / BKV, Hq, B);
  flash_bwd_dkv_kernel<<<grid, THREADS, SmemK::TOTAL, (cudaStream_t)stream>>>(tmQ, tmdO, tmK, tmV, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
