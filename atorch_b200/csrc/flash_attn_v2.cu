// Flash attention forward, two query tiles per CTA (head dim 128, bf16) for sm_100a.
//
// One CTA owns 256 query rows as two 128-row tiles A and B that share every K/V tile. Warp 0 = TMA
// producer, warp 1 = MMA issuer / TMEM owner, warps 2..5 = softmax of tile A, warps 6..9 = softmax of
// tile B; a softmax thread owns one whole row (128 scores), so no row statistics are exchanged.
//
//   TMEM:  S_A | S_B | O_A | O_B   (4 x 128 fp32 columns); P_T (bf16) overwrites the first 64 columns of S_T
//   per K/V tile j:   S_T = Q_T K_j^T  ->  P_T = 2^(S_T c - m_T c)  ->  O_T += P_T V_j
//
// P never leaves tensor memory: the softmax thread stores its packed row with tcgen05.st and the P.V
// product reads it as the A operand of tcgen05.mma. O accumulates in tensor memory. The reference maximum
// m_T of a row is only raised when the new row maximum exceeds it by more than 2^8 (in the exponent
// domain); then the row of O_T is rescaled in TMEM by the owning thread, which is safe because the scores
// S_T(j) it has just waited for were issued after the product P_T(j-1) V and complete after it.
// While tile A's warps exponentiate, the tensor core works for tile B and vice versa:
// issue order  PV_A(j), S_A(j+1), PV_B(j), S_B(j+1).
//
// Masks: per-row key interval [lo, hi) exactly as in flash_attn.cu; each query tile walks only the K/V
// tiles up to the last one that any of its rows can see.
#include "common.cuh"
#include <type_traits>

namespace {
using namespace atb;

constexpr int BQ = 128, BKV = 128, HD = 128;
constexpr int PANEL = 128 * 64 * 2;
constexpr int TILE = 2 * PANEL;
constexpr int THREADS = 64 + 256;
constexpr float RESCALE_THRESHOLD = 8.f;   // log2 units

struct Params {
  __nv_bfloat16* O;
  float* lse;
  const int* row_lo;
  const int* row_hi;
  int B, Sq, Sk, Hq, Hkv, causal;
  float scale_log2;
  int* status;
};

struct L2 {
  static constexpr int Q_OFF = 0;                    // tile A, tile B
  static constexpr int K_OFF = Q_OFF + 2 * TILE;     // 2 stages
  static constexpr int V_OFF = K_OFF + 2 * TILE;     // 2 stages
  static constexpr int BAR_OFF = V_OFF + 2 * TILE;   // 192 KB
  static constexpr int NBARS = 1 + 8 + 2 + 2 + 2;
  static constexpr int TOTAL = BAR_OFF + NBARS * 8 + 64 + 1024;
};

// P = 2^(S c - m c) for one row: the 128 scores are read back from tensor memory in chunks of 32 (the next
// chunk's load is in flight while this one is exponentiated) and the packed bf16 result overwrites the first
// 64 columns of S; each chunk is read before the 16 columns it turns into are written, and those lie below
// the next chunk. Returns the row sum. MASK: per-element key interval test (tiles that are not fully visible).
template <bool MASK>
ATB_DEVICE float softmax_exp_row(uint32_t s_addr, float scale_log2, float neg_ms, int kv0, int lo, int hi) {
  const uint64_t sc2 = f2_pack(scale_log2, scale_log2), nm2 = f2_pack(neg_ms, neg_ms);
  uint64_t acc0 = 0ull, acc1 = 0ull;   // (0.f, 0.f)
  uint32_t xa[32], xb[32];
  tmem_ld_32x32(s_addr, xa);
#pragma unroll
  for (int cc = 0; cc < 4; ++cc) {
    uint32_t (&x)[32] = (cc & 1) ? xb : xa;
    uint32_t (&xn)[32] = (cc & 1) ? xa : xb;
    tmem_ld_wait();
    if (cc + 1 < 4) tmem_ld_32x32(s_addr + (cc + 1) * 32, xn);
    uint32_t pk[16];
#pragma unroll
    for (int c = 0; c < 32; c += 2) {
      float t0, t1;
      f2_unpack(f2_fma(f2_pack_bits(x[c], x[c + 1]), sc2, nm2), t0, t1);
      float p0 = fast_exp2(t0), p1 = fast_exp2(t1);
      if (MASK) {
        const int kk = kv0 + cc * 32 + c;
        if (kk < lo || kk >= hi) p0 = 0.f;
        if (kk + 1 < lo || kk + 1 >= hi) p1 = 0.f;
      }
      const uint64_t pp = f2_pack(p0, p1);
      if ((c >> 1) & 1) acc1 = f2_add(acc1, pp);
      else acc0 = f2_add(acc0, pp);
      pk[c >> 1] = pack_bf16x2(p0, p1);
    }
    tmem_st_32x16(s_addr + cc * 16, pk);
  }
  float a, b, c, d;
  f2_unpack(acc0, a, b);
  f2_unpack(acc1, c, d);
  return (a + b) + (c + d);
}

__global__ void __launch_bounds__(THREADS, 1)
flash_fwd2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                  const __grid_constant__ CUtensorMap tmV, Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + L2::Q_OFF;
  uint8_t* sK = smem + L2::K_OFF;
  uint8_t* sV = smem + L2::V_OFF;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L2::BAR_OFF);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;      // [2]
  uint64_t* k_empty = bars + 3;     // [2]
  uint64_t* v_full = bars + 5;      // [2]
  uint64_t* v_empty = bars + 7;     // [2]
  uint64_t* s_full = bars + 9;      // [2] per query tile: S_T(j) is in TMEM (and P_T(j-1) V has completed)
  uint64_t* p_full = bars + 11;     // [2] per query tile: P_T(j) is in TMEM
  uint64_t* o_full = bars + 13;     // [2] per query tile: the last P.V product has completed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + L2::NBARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* kv_range = const_cast<int*>(reinterpret_cast<volatile int*>(tmem_slot + 2));  // t0, t1 of tile A, t1 of tile B

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != 0) return;
  const int qb = gridDim.x - 1 - blockIdx.x;
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.Hq / p.Hkv);
  const int q0 = qb * 2 * BQ;
  const int shift = p.Sk - p.Sq;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1); mbar_init(&p_full[i], 4); mbar_init(&o_full[i], 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc<1>(tmem_slot, 512); tmem_relinquish<1>(); }
  if (warp == 2) {   // union of the key intervals of the rows of each tile
    int umin[2] = {INT_MAX, INT_MAX}, umax[2] = {0, 0};
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      for (int r = lane; r < BQ; r += 32) {
        const int i = q0 + t * BQ + r;
        if (i >= p.Sq) continue;
        int lo = p.row_lo ? p.row_lo[(long long)b * p.Sq + i] : 0;
        int hi = p.row_hi ? p.row_hi[(long long)b * p.Sq + i] : (p.causal ? i + 1 + shift : p.Sk);
        lo = max(lo, 0); hi = min(hi, p.Sk);
        if (hi > lo) { umin[t] = min(umin[t], lo); umax[t] = max(umax[t], hi); }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        umin[t] = min(umin[t], __shfl_xor_sync(0xffffffffu, umin[t], o));
        umax[t] = max(umax[t], __shfl_xor_sync(0xffffffffu, umax[t], o));
      }
    }
    if (lane == 0) {
      const int lo = min(umin[0], umin[1]);
      const int first = lo == INT_MAX ? 0 : lo / BKV;
      kv_range[0] = first;
      kv_range[1] = umax[0] > umin[0] ? (umax[0] + BKV - 1) / BKV : first;
      kv_range[2] = umax[1] > umin[1] ? (umax[1] + BKV - 1) / BKV : first;
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int t0 = kv_range[0];
  const int n_a = kv_range[1] - t0, n_b = kv_range[2] - t0;   // K/V tiles of query tile A / B
  const int n = max(n_a, n_b);
  const long long q_row0 = (long long)b * p.Sq + q0;
  const long long k_row0 = (long long)b * p.Sk;

  if (warp == 0) {
    if (lane == 0 && n > 0) {
      tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
      mbar_expect_tx(q_full, 2 * TILE);
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        tma_load_2d(sQ + t * TILE, &tmQ, q_full, h * HD, (int)(q_row0 + t * BQ));
        tma_load_2d(sQ + t * TILE + PANEL, &tmQ, q_full, h * HD + 64, (int)(q_row0 + t * BQ));
      }
      for (int j = 0; j < n; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const int krow = (int)(k_row0 + (long long)(t0 + j) * BKV);
        if (!mbar_wait(&k_empty[s], ph ^ 1, abort_flag, p.status)) break;
        mbar_expect_tx(&k_full[s], TILE);
        tma_load_2d(sK + s * TILE, &tmK, &k_full[s], hk * HD, krow);
        tma_load_2d(sK + s * TILE + PANEL, &tmK, &k_full[s], hk * HD + 64, krow);
        if (!mbar_wait(&v_empty[s], ph ^ 1, abort_flag, p.status)) break;
        mbar_expect_tx(&v_full[s], TILE);
        tma_load_2d(sV + s * TILE, &tmV, &v_full[s], hk * HD, krow);
        tma_load_2d(sV + s * TILE + PANEL, &tmV, &v_full[s], hk * HD + 64, krow);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n > 0) {
      constexpr uint32_t idesc_s = umma_idesc(BQ, BKV, 1, 1, false, false);
      constexpr uint32_t idesc_o = umma_idesc(BQ, HD, 1, 1, false, true);
      int k_ready = -1, v_ready = -1;   // newest K / V tile whose arrival has been waited for
      // descriptors of the tiles' first MMA operands; the loops below only advance them
      // (kept in scalars and picked with selects: an array indexed at run time would live in local memory)
      const uint64_t q_desc0 = umma_desc_sw128(smem_u32(sQ), 16, 1024), k_desc0 = umma_desc_sw128(smem_u32(sK), 16, 1024),
                     v_desc0 = umma_desc_sw128(smem_u32(sV), PANEL, 1024);
      // S_T(j) = Q_T K_j^T into the tile's S columns
      auto issue_s = [&](int t, int j) -> bool {
        const int s = j & 1;
        if (k_ready < j) {
          if (!mbar_wait(&k_full[s], (j >> 1) & 1, abort_flag, p.status)) return false;
          k_ready = j;
          tc_fence_after();
        }
        const uint64_t qd = umma_desc_advance(q_desc0, t ? TILE : 0), kd = umma_desc_advance(k_desc0, s ? TILE : 0);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t off = (k >> 2) * PANEL + (k & 3) * 32;
          umma_f16<1>(tmem_base + t * BKV, umma_desc_advance(qd, off), umma_desc_advance(kd, off), idesc_s, k != 0);
        }
        umma_commit(&s_full[t]);
        return true;
      };
      bool ok = mbar_wait(q_full, 0, abort_flag, p.status);
      if (ok && n_a > 0) ok = issue_s(0, 0);
      if (ok && n_b > 0) ok = issue_s(1, 0);
      if (ok) umma_commit(&k_empty[0]);
      // one half-step of the ping-pong for query tile T (compile-time, so that nothing is indexed at run time):
      // P_T(j) V_j into O_T, then the next scores S_T(j+1)
      auto half_step = [&](auto tile, int j) -> bool {
        constexpr int t = decltype(tile)::value;
        const int n_t = t ? n_b : n_a;
        const int s = j & 1;
        if (j < n_t) {
          if (!mbar_wait(&p_full[t], j & 1, abort_flag, p.status)) return false;
          if (v_ready < j) {
            if (!mbar_wait(&v_full[s], (j >> 1) & 1, abort_flag, p.status)) return false;
            v_ready = j;
          }
          tc_fence_after();
          const uint64_t vd = umma_desc_advance(v_desc0, s ? TILE : 0);
#pragma unroll
          for (int k = 0; k < BKV / 16; ++k)   // A = P_T: 16 bf16 keys per step = 8 TMEM columns
            umma_f16_ts(tmem_base + 2 * BKV + t * HD, tmem_base + t * BKV + k * 8, umma_desc_advance(vd, k * 2048),
                        idesc_o, (j | k) != 0);
          if (j == n_t - 1) umma_commit(&o_full[t]);
        }
        if (t == 1) umma_commit(&v_empty[s]);
        if (j + 1 < n_t && !issue_s(t, j + 1)) return false;
        if (t == 1 && j + 1 < n) umma_commit(&k_empty[(j + 1) & 1]);
        return true;
      };
      for (int j = 0; ok && j < n; ++j)
        ok = half_step(std::integral_constant<int, 0>{}, j) && half_step(std::integral_constant<int, 1>{}, j);
    }
  } else {
    const int t = (warp - 2) >> 2;            // query tile of this warp
    const int quarter = warp & 3;             // TMEM lane quarter
    const int r = quarter * 32 + lane;        // row inside the tile
    const int i = q0 + t * BQ + r;            // global query row
    const bool row_valid = i < p.Sq;
    const int n_t = t ? n_b : n_a;
    int lo = 0, hi = 0;
    if (row_valid) {
      lo = p.row_lo ? p.row_lo[(long long)b * p.Sq + i] : 0;
      hi = p.row_hi ? p.row_hi[(long long)b * p.Sq + i] : (p.causal ? i + 1 + shift : p.Sk);
      lo = max(lo, 0); hi = min(hi, p.Sk);
    }
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const uint32_t s_addr = lane_addr + t * BKV, o_addr = lane_addr + 2 * BKV + t * HD;
    float m_ref = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < n_t; ++j) {
      const int kv0 = (t0 + j) * BKV;
      if (!__all_sync(0xffffffffu, mbar_wait(&s_full[t], j & 1, abort_flag, p.status))) { ok = false; break; }
      tc_fence_after();
      // the mask tests are compiled into a separate path taken only by warps with a partly visible row
      const bool full = __all_sync(0xffffffffu, row_valid && lo <= kv0 && hi >= kv0 + BKV);
      // ---- pass 1: row maximum
      float mx;
      {
        uint32_t x0[32], x1[32], x2[32], x3[32];
        tmem_ld_32x32(s_addr, x0);
        tmem_ld_32x32(s_addr + 32, x1);
        tmem_ld_32x32(s_addr + 64, x2);
        tmem_ld_32x32(s_addr + 96, x3);
        tmem_ld_wait();
        if (!full) {
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            if (kv0 + c < lo || kv0 + c >= hi) x0[c] = 0xff800000u;
            if (kv0 + 32 + c < lo || kv0 + 32 + c >= hi) x1[c] = 0xff800000u;
            if (kv0 + 64 + c < lo || kv0 + 64 + c >= hi) x2[c] = 0xff800000u;
            if (kv0 + 96 + c < lo || kv0 + 96 + c >= hi) x3[c] = 0xff800000u;
          }
        }
        float m4[4] = {__uint_as_float(x0[0]), __uint_as_float(x1[0]), __uint_as_float(x2[0]), __uint_as_float(x3[0])};
#pragma unroll
        for (int c = 1; c < 32; ++c) {
          m4[0] = fmaxf(m4[0], __uint_as_float(x0[c])); m4[1] = fmaxf(m4[1], __uint_as_float(x1[c]));
          m4[2] = fmaxf(m4[2], __uint_as_float(x2[c])); m4[3] = fmaxf(m4[3], __uint_as_float(x3[c]));
        }
        mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
      }
      // raise the reference maximum only when it pays: a stale one costs nothing while 2^(gap) fits bf16/fp32
      const bool raise = (mx > m_ref) && (m_ref == -INFINITY || (mx - m_ref) * p.scale_log2 > RESCALE_THRESHOLD);
      if (__any_sync(0xffffffffu, raise)) {
        float alpha = 1.f;
        if (raise) {
          alpha = (m_ref == -INFINITY) ? 0.f : fast_exp2((m_ref - mx) * p.scale_log2);
          m_ref = mx;
          l_run *= alpha;
        }
        if (j > 0) {   // O_T holds the products up to tile j-1 (complete: S_T(j) was issued after them)
#pragma unroll
          for (int cc = 0; cc < 4; ++cc) {
            uint32_t tr[32];
            tmem_ld_32x32(o_addr + cc * 32, tr);
            tmem_ld_wait();
#pragma unroll
            for (int c = 0; c < 32; ++c) tr[c] = __float_as_uint(__uint_as_float(tr[c]) * alpha);
            tmem_st_32x32(o_addr + cc * 32, tr);
          }
        }
      }
      // ---- pass 2: P = 2^(S c - m c) as packed bf16 over the first 64 columns of S
      const float neg_ms = (m_ref == -INFINITY) ? 0.f : -m_ref * p.scale_log2;
      l_run += full ? softmax_exp_row<false>(s_addr, p.scale_log2, neg_ms, kv0, lo, hi)
                    : softmax_exp_row<true>(s_addr, p.scale_log2, neg_ms, kv0, lo, hi);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[t]);
    }
    if (ok && n_t > 0) ok = __all_sync(0xffffffffu, mbar_wait(&o_full[t], 0, abort_flag, p.status));
    if (ok) {
      if (n_t > 0) tc_fence_after();
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      __nv_bfloat16* orow = p.O + (((long long)b * p.Sq + i) * p.Hq + h) * HD;
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) {
        uint32_t tr[32];
        if (n_t > 0) {
          tmem_ld_32x32(o_addr + cc * 32, tr);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int c = 0; c < 32; ++c) tr[c] = 0u;
        }
        if (row_valid) {
#pragma unroll
          for (int c = 0; c < 32; c += 8) {
            uint4 v;
            v.x = pack_bf16x2(__uint_as_float(tr[c]) * inv, __uint_as_float(tr[c + 1]) * inv);
            v.y = pack_bf16x2(__uint_as_float(tr[c + 2]) * inv, __uint_as_float(tr[c + 3]) * inv);
            v.z = pack_bf16x2(__uint_as_float(tr[c + 4]) * inv, __uint_as_float(tr[c + 5]) * inv);
            v.w = pack_bf16x2(__uint_as_float(tr[c + 6]) * inv, __uint_as_float(tr[c + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + cc * 32 + c) = v;
          }
        }
      }
      if (row_valid)
        p.lse[((long long)b * p.Hq + h) * p.Sq + i] =
            l_run > 0.f ? (m_ref * p.scale_log2 + log2f(l_run)) * 0.6931471805599453f : -INFINITY;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    const uint64_t t_start = globaltimer_ns();
    while (globaltimer_ns() - t_start < 200000ull) __nanosleep(1000);
  }
  if (warp == 1) { tc_fence_after(); tmem_dealloc<1>(tmem_base, 512); }
}

}  // namespace

// Same contract as atb_flash_fwd (flash_attn.cu).
extern "C" int atb_flash_fwd_v2(const void* q, const void* k, const void* v, void* o, float* lse, const int* row_lo,
                                const int* row_hi, int B, int Sq, int Sk, int Hq, int Hkv, long long q_stride,
                                long long k_stride, long long v_stride, int causal, float softmax_scale, void* stream,
                                int* status) {
  if (B <= 0 || Sq <= 0 || Sk <= 0) return 0;
  if (Hq % Hkv) return -1;
  if ((q_stride | k_stride | v_stride) & 7) return -1;
  CUtensorMap tmQ, tmK, tmV;
  if (!make_tmap_2d(&tmQ, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)B * Sq, (uint64_t)Hq * HD, q_stride, BQ,
                    64, CU_TENSOR_MAP_SWIZZLE_128B))
    return -2;
  if (!make_tmap_2d(&tmK, k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)B * Sk, (uint64_t)Hkv * HD, k_stride,
                    BKV, 64, CU_TENSOR_MAP_SWIZZLE_128B))
    return -2;
  if (!make_tmap_2d(&tmV, v, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)B * Sk, (uint64_t)Hkv * HD, v_stride,
                    BKV, 64, CU_TENSOR_MAP_SWIZZLE_128B))
    return -2;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(flash_fwd2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L2::TOTAL) != cudaSuccess)
      return -4;
    attr_set = true;
  }
  Params p;
  p.O = (__nv_bfloat16*)o; p.lse = lse; p.row_lo = row_lo; p.row_hi = row_hi;
  p.B = B; p.Sq = Sq; p.Sk = Sk; p.Hq = Hq; p.Hkv = Hkv; p.causal = causal;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.status = status;
  dim3 grid((Sq + 2 * BQ - 1) / (2 * BQ), Hq, B);
  flash_fwd2_kernel<<<grid, THREADS, L2::TOTAL, (cudaStream_t)stream>>>(tmQ, tmK, tmV, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
