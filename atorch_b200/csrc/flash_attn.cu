// Flash attention forward for sm_100a (head dim 128 or 64, bf16), tcgen05 + TMEM + TMA.
//
// One CTA per (128 query rows, head, batch). Warp 0 = TMA producer, warp 1 = MMA issuer and TMEM
// owner, warps 2..9 = softmax: two warps per TMEM lane quarter, thread (row r, half h) owns
// columns [64h, 64h+64) of row r of the score tile and of the output tile.
//
//   S_j   = Q K_j^T                       tcgen05.mma  smem x smem -> TMEM (two S buffers)
//   P_j   = exp2(S_j * c - m)             registers; written as bf16 into swizzled shared memory
//   O_j   = P_j V_j                       tcgen05.mma  smem x smem -> TMEM (fresh tile)
//   O    := O * alpha_j + O_j             registers (fp32), final O / l and lse = m + log(l)
//
// The MMA warp issues S_{j+1} before P_j V_j, so the tensor core works on the next scores while
// the softmax warps exponentiate the current ones.
//
// Masks: every mask of the front end is a per-row key interval [lo, hi): causal (hi = i+1 + Sk-Sq),
// GLM break-point (hi = max(i+1, g[b])), packed GLM (hi = max over spans), key padding (hi capped
// by the key length), packed variable-length sequences (lo = start of the row's sequence).
// `row_lo` / `row_hi` (int32 [B, Sq], either may be null) carry the explicit form; KV tiles outside
// the union of the block's intervals are skipped and tiles inside their intersection are
// processed without per-element tests.
//
// Replaces flash_attn_func / flash_attn_varlen_func (FA2 sm_80 kernels) behind FlashAttnModule in
// the reference (atorch/modules/transformer/layers.py:1283-1408).
#include "common.cuh"

namespace {
using namespace atb;

constexpr int BQ = 128;   // query rows per CTA
constexpr int BKV = 128;  // keys per tile
constexpr int HD = 128;   // head dim
constexpr int PANEL = BQ * 64 * 2;  // bytes of one [128 x 64] bf16 panel (16 KB)
constexpr int TILE = 2 * PANEL;     // [128 x 128] bf16 tile (32 KB)
constexpr int KV_STAGES = 2;
constexpr int N_SOFTMAX = 256;
constexpr int THREADS = 64 + N_SOFTMAX;

struct FwdParams {
  __nv_bfloat16* O;   // [B, Sq, Hq, HD] contiguous
  float* lse;         // [B, Hq, Sq]
  const int* row_lo;  // [B, Sq] or null
  const int* row_hi;  // [B, Sq] or null
  int B, Sq, Sk, Hq, Hkv;
  int causal;         // analytic causal bound when row_hi is null
  float scale_log2;   // softmax scale * log2(e)
  int* status;
  DropParams drop;    // attention dropout (thr16 == 0: none)
  BiasParams bias;    // additive bias on the scaled scores (ptr == nullptr: none)
  float inv_scale;    // 1 / softmax scale: the bias is folded into the raw scores
};

struct SmemLayout {
  static constexpr int Q_OFF = 0;
  static constexpr int K_OFF = Q_OFF + TILE;
  static constexpr int V_OFF = K_OFF + KV_STAGES * TILE;
  static constexpr int P_OFF = V_OFF + KV_STAGES * TILE;
  static constexpr int MISC_OFF = P_OFF + TILE;                  // 192 KB so far
  static constexpr int ROWMAX_OFF = MISC_OFF;                    // float [2][2][128]
  static constexpr int ROWSUM_OFF = ROWMAX_OFF + 2 * 2 * 128 * 4;  // float [2][128]
  static constexpr int BAR_OFF = ROWSUM_OFF + 2 * 128 * 4;
  static constexpr int NBARS = 1 + 4 * KV_STAGES + 2 + 2 + 4;
  static constexpr int TOTAL = BAR_OFF + NBARS * 8 + 64 + 1024;
};

// HDIM = 128 or 64: with 64 the Q / K / V tiles are one 64-column panel (in the same shared-memory slots), the
// score product runs over four k-steps and the output tile has 64 columns, 32 per thread.
template <bool DROP, bool BIAS, int HDIM = 128>
__global__ void __launch_bounds__(THREADS, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, FwdParams p) {
  using L = SmemLayout;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + L::Q_OFF;
  uint8_t* sK = smem + L::K_OFF;
  uint8_t* sV = smem + L::V_OFF;
  uint8_t* sP = smem + L::P_OFF;
  float* s_rowmax = reinterpret_cast<float*>(smem + L::ROWMAX_OFF);
  float* s_rowsum = reinterpret_cast<float*>(smem + L::ROWSUM_OFF);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;
  uint64_t* k_empty = k_full + KV_STAGES;
  uint64_t* v_full = k_empty + KV_STAGES;
  uint64_t* v_empty = v_full + KV_STAGES;
  uint64_t* s_full = v_empty + KV_STAGES;  // [2]
  uint64_t* s_free = s_full + 2;           // [2]
  uint64_t* p_full = s_free + 2;
  uint64_t* p_free = p_full + 1;
  uint64_t* o_full = p_free + 1;
  uint64_t* x_bar = o_full + 1;  // row statistics exchanged between the two halves of a row
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(x_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* kv_range = const_cast<int*>(reinterpret_cast<volatile int*>(tmem_slot + 2));  // [4]: t0, t1, full_lo, full_hi

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // a wait already ran out somewhere in this stream of work: do not start, so that a failing
  // launch ends after one wait limit instead of one per wave of CTAs
  if (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != 0) return;
  const int qb = gridDim.x - 1 - blockIdx.x;  // heaviest (last) causal blocks first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.Hq / p.Hkv);
  const int q0 = qb * BQ;
  const int causal_shift = p.Sk - p.Sq;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < KV_STAGES; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&s_free[i], N_SOFTMAX / 32);
    }
    mbar_init(p_full, N_SOFTMAX / 32);
    mbar_init(p_free, 1);
    mbar_init(o_full, 1);
    mbar_init(x_bar, N_SOFTMAX / 32);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc<1>(tmem_slot, 512);
    tmem_relinquish<1>();
  }
  // Key range of this query block: union [umin, umax) and intersection [imax_lo, imin_hi) of the
  // rows' intervals, reduced by warp 2.
  if (warp == 2) {
    int umin = INT_MAX, umax = 0, ilo = 0, ihi = INT_MAX;
    for (int r = lane; r < BQ; r += 32) {
      const int i = q0 + r;
      if (i >= p.Sq) continue;
      int lo = p.row_lo ? p.row_lo[(long long)b * p.Sq + i] : 0;
      int hi = p.row_hi ? p.row_hi[(long long)b * p.Sq + i] : (p.causal ? i + 1 + causal_shift : p.Sk);
      lo = max(lo, 0);
      hi = min(hi, p.Sk);
      if (hi <= lo) { ilo = INT_MAX; ihi = 0; continue; }
      umin = min(umin, lo); umax = max(umax, hi);
      ilo = max(ilo, lo); ihi = min(ihi, hi);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      umin = min(umin, __shfl_xor_sync(0xffffffffu, umin, o));
      umax = max(umax, __shfl_xor_sync(0xffffffffu, umax, o));
      ilo = max(ilo, __shfl_xor_sync(0xffffffffu, ilo, o));
      ihi = min(ihi, __shfl_xor_sync(0xffffffffu, ihi, o));
    }
    if (lane == 0) {
      kv_range[0] = umax > umin ? umin / BKV : 0;
      kv_range[1] = umax > umin ? (umax + BKV - 1) / BKV : 0;
      kv_range[2] = ilo;
      kv_range[3] = ihi;
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int t0 = kv_range[0], t1 = kv_range[1];
  const int full_lo = kv_range[2], full_hi = kv_range[3];
  const int ntiles = t1 - t0;
  const long long q_row0 = (long long)b * p.Sq + q0;
  const long long k_row0 = (long long)b * p.Sk;

  if (warp == 0) {
    if (lane == 0 && ntiles > 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      constexpr int TILE_B = (HDIM / 64) * PANEL;   // bytes of a [128 x HDIM] tile
      mbar_expect_tx(q_full, TILE_B);
      tma_load_2d(sQ, &tmQ, q_full, h * HDIM, (int)q_row0);
      if (HDIM == 128) tma_load_2d(sQ + PANEL, &tmQ, q_full, h * HDIM + 64, (int)q_row0);
      for (int j = 0; j < ntiles; ++j) {
        const int s = j % KV_STAGES;
        const uint32_t ph = (j / KV_STAGES) & 1;
        const int krow = (int)(k_row0 + (long long)(t0 + j) * BKV);
        if (!mbar_wait(&k_empty[s], ph ^ 1, abort_flag, p.status)) break;
        mbar_expect_tx(&k_full[s], TILE_B);
        tma_load_2d(sK + s * TILE, &tmK, &k_full[s], hk * HDIM, krow);
        if (HDIM == 128) tma_load_2d(sK + s * TILE + PANEL, &tmK, &k_full[s], hk * HDIM + 64, krow);
        if (!mbar_wait(&v_empty[s], ph ^ 1, abort_flag, p.status)) break;
        mbar_expect_tx(&v_full[s], TILE_B);
        tma_load_2d(sV + s * TILE, &tmV, &v_full[s], hk * HDIM, krow);
        if (HDIM == 128) tma_load_2d(sV + s * TILE + PANEL, &tmV, &v_full[s], hk * HDIM + 64, krow);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && ntiles > 0) {
      constexpr uint32_t idesc_s = umma_idesc(BQ, BKV, 1, 1, false, false);
      constexpr uint32_t idesc_o = umma_idesc(BQ, HDIM, 1, 1, false, true);
      const uint32_t q_addr = smem_u32(sQ), p_addr = smem_u32(sP);
      auto issue_s = [&](int j) -> bool {
        const int s = j % KV_STAGES, sb = j & 1;
        if (!mbar_wait(&k_full[s], (j / KV_STAGES) & 1, abort_flag, p.status)) return false;
        if (!mbar_wait(&s_free[sb], ((j >> 1) & 1) ^ 1, abort_flag, p.status)) return false;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(sK + s * TILE);
#pragma unroll
        for (int k = 0; k < HDIM / 16; ++k) {
          const uint32_t off = (k >> 2) * PANEL + (k & 3) * 32;
          umma_f16<1>(tmem_base + sb * BKV, umma_desc_sw128(q_addr + off, 16, 1024),
                      umma_desc_sw128(k_addr + off, 16, 1024), idesc_s, k != 0);
        }
        umma_commit(&s_full[sb]);
        umma_commit(&k_empty[s]);
        return true;
      };
      bool ok = mbar_wait(q_full, 0, abort_flag, p.status);
      ok = ok && issue_s(0);
      for (int j = 0; ok && j < ntiles; ++j) {
        if (j + 1 < ntiles) ok = issue_s(j + 1);
        if (!ok) break;
        const int s = j % KV_STAGES;
        if (!mbar_wait(p_full, j & 1, abort_flag, p.status)) break;
        if (!mbar_wait(&v_full[s], (j / KV_STAGES) & 1, abort_flag, p.status)) break;
        tc_fence_after();
        const uint32_t v_addr = smem_u32(sV + s * TILE);
#pragma unroll
        for (int k = 0; k < BKV / 16; ++k) {
          const uint32_t a_off = (k >> 2) * PANEL + (k & 3) * 32;
          umma_f16<1>(tmem_base + 2 * BKV, umma_desc_sw128(p_addr + a_off, 16, 1024),
                      umma_desc_sw128(v_addr + k * 2048, PANEL, 1024), idesc_o, k != 0);
        }
        umma_commit(o_full);
        umma_commit(&v_empty[s]);
        umma_commit(p_free);
      }
    }
  } else {
    // ------------------------------ softmax / output warps ------------------------------
    const int sw = warp - 2;          // 0..7
    const int quarter = warp & 3;     // TMEM lane quarter this warp may touch
    const int half = sw >> 2;         // which 64-column half of the tiles this thread owns
    const int r = quarter * 32 + lane;
    const int i = q0 + r;             // global query row
    const bool row_valid = i < p.Sq;
    int lo = 0, hi = 0;
    if (row_valid) {
      lo = p.row_lo ? p.row_lo[(long long)b * p.Sq + i] : 0;
      hi = p.row_hi ? p.row_hi[(long long)b * p.Sq + i] : (p.causal ? i + 1 + causal_shift : p.Sk);
      lo = max(lo, 0);
      hi = min(hi, p.Sk);
    }
    float m_run = -INFINITY, l_run = 0.f, alpha_prev = 1.f;
    const uint32_t drop_key = DROP ? drop_row_key(p.drop, (uint32_t)(b * p.Hq + h), (uint32_t)i) : 0u;
    float o_acc[64];
#pragma unroll
    for (int c = 0; c < 64; ++c) o_acc[c] = 0.f;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    bool ok = true;

    auto accumulate_o = [&](int j) -> bool {  // O := O * alpha_j + O_j
      if (!__all_sync(0xffffffffu, mbar_wait(o_full, j & 1, abort_flag, p.status))) return false;
      tc_fence_after();
#pragma unroll
      for (int cc = 0; cc < HDIM / 64; ++cc) {
        uint32_t t[32];
        tmem_ld_32x32(lane_addr + 2 * BKV + half * (HDIM / 2) + cc * 32, t);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 32; ++c) o_acc[cc * 32 + c] = o_acc[cc * 32 + c] * alpha_prev + __uint_as_float(t[c]);
      }
      return true;
    };

    for (int j = 0; j < ntiles; ++j) {
      const int sb = j & 1;
      const int kv0 = (t0 + j) * BKV;
      if (!__all_sync(0xffffffffu, mbar_wait(&s_full[sb], (j >> 1) & 1, abort_flag, p.status))) { ok = false; break; }
      tc_fence_after();
      float sv[64];
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        uint32_t t[32];
        tmem_ld_32x32(lane_addr + sb * BKV + half * 64 + cc * 32, t);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 32; ++c) sv[cc * 32 + c] = __uint_as_float(t[c]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_free[sb]);
      if constexpr (BIAS) {
        // s + bias / scale, so that the scale folded into the exponent leaves the bias as given
        if (row_valid) {
          const int cb = kv0 + half * 64;
          const __nv_bfloat16* bp = p.bias.ptr + (long long)b * p.bias.sb + (long long)h * p.bias.sh +
                                    (long long)i * p.bias.sq + cb;
#pragma unroll
          for (int c8 = 0; c8 < 8; ++c8) {
            if (cb + c8 * 8 < p.Sk) {
              const uint4 u = *reinterpret_cast<const uint4*>(bp + c8 * 8);
              const float2 b0 = unpack_bf16x2(u.x), b1 = unpack_bf16x2(u.y), b2 = unpack_bf16x2(u.z),
                           b3 = unpack_bf16x2(u.w);
              float* d = sv + c8 * 8;
              d[0] = fmaf(b0.x, p.inv_scale, d[0]); d[1] = fmaf(b0.y, p.inv_scale, d[1]);
              d[2] = fmaf(b1.x, p.inv_scale, d[2]); d[3] = fmaf(b1.y, p.inv_scale, d[3]);
              d[4] = fmaf(b2.x, p.inv_scale, d[4]); d[5] = fmaf(b2.y, p.inv_scale, d[5]);
              d[6] = fmaf(b3.x, p.inv_scale, d[6]); d[7] = fmaf(b3.y, p.inv_scale, d[7]);
            }
          }
        }
      }
      const bool tile_full = (kv0 >= full_lo) && (kv0 + BKV <= full_hi);
      if (!tile_full) {
        const int c0 = kv0 + half * 64;
#pragma unroll
        for (int c = 0; c < 64; ++c) {
          const int jj = c0 + c;
          if (jj < lo || jj >= hi) sv[c] = -INFINITY;
        }
      }
      // four independent chains instead of one chain of 63 dependent max operations
      float mx4[4] = {sv[0], sv[1], sv[2], sv[3]};
#pragma unroll
      for (int c = 4; c < 64; c += 4) {
        mx4[0] = fmaxf(mx4[0], sv[c]); mx4[1] = fmaxf(mx4[1], sv[c + 1]);
        mx4[2] = fmaxf(mx4[2], sv[c + 2]); mx4[3] = fmaxf(mx4[3], sv[c + 3]);
      }
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      float* rm = s_rowmax + (j & 1) * 256;
      rm[half * 128 + r] = mx;
      __syncwarp();
      if (lane == 0) mbar_arrive(x_bar);
      if (!__all_sync(0xffffffffu, mbar_wait(x_bar, j & 1, abort_flag, p.status))) { ok = false; break; }
      mx = fmaxf(mx, rm[(half ^ 1) * 128 + r]);
      // m_run / mx are raw (unscaled) score maxima; the softmax scale (> 0) is folded into the
      // exponent: p = 2^(s * c - m * c), one FFMA + one EX2 per element
      const float m_new = fmaxf(m_run, mx);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = fast_exp2((m_run - m_use) * p.scale_log2);  // m_run = -inf -> 0
      const float neg_ms = -m_use * p.scale_log2;
      float ls4[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t pk[32];
      if constexpr (!DROP) {
#pragma unroll
        for (int c = 0; c < 64; c += 2) {
          const float p0 = fast_exp2(fmaf(sv[c], p.scale_log2, neg_ms));
          const float p1 = fast_exp2(fmaf(sv[c + 1], p.scale_log2, neg_ms));
          ls4[(c >> 1) & 3] += p0 + p1;
          pk[c >> 1] = pack_bf16x2(p0, p1);
        }
      } else {
        // the row sum (and lse) is that of the full softmax; dropped elements only leave the P V product,
        // and the 1 / (1 - p) factor is applied once, to the finished row
        const uint32_t cbase = (uint32_t)(kv0 + half * 64);
#pragma unroll
        for (int c = 0; c < 64; c += 2) {
          const float p0 = fast_exp2(fmaf(sv[c], p.scale_log2, neg_ms));
          const float p1 = fast_exp2(fmaf(sv[c + 1], p.scale_log2, neg_ms));
          ls4[(c >> 1) & 3] += p0 + p1;
          const uint32_t w = drop_pair_bits(drop_key, cbase + c);
          pk[c >> 1] = pack_bf16x2((w & 0xffffu) >= p.drop.thr16 ? p0 : 0.f, (w >> 16) >= p.drop.thr16 ? p1 : 0.f);
        }
      }
      l_run = l_run * alpha + ((ls4[0] + ls4[1]) + (ls4[2] + ls4[3]));
      m_run = m_new;
      // previous tile's P V product must be folded in (and must have finished reading sP)
      if (j > 0) {
        if (!accumulate_o(j - 1)) { ok = false; break; }
        if (!__all_sync(0xffffffffu, mbar_wait(p_free, (j - 1) & 1, abort_flag, p.status))) { ok = false; break; }
      }
      alpha_prev = alpha;
      // P tile, K-major 128B-swizzled: panel `half`, row r, 16-byte chunk c8 at slot (c8 ^ (r & 7))
      uint8_t* prow = sP + half * PANEL + r * 128;
#pragma unroll
      for (int c8 = 0; c8 < 8; ++c8) {
        uint4 v = make_uint4(pk[c8 * 4], pk[c8 * 4 + 1], pk[c8 * 4 + 2], pk[c8 * 4 + 3]);
        *reinterpret_cast<uint4*>(prow + ((c8 ^ (r & 7)) << 4)) = v;
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    if (ok && ntiles > 0) ok = accumulate_o(ntiles - 1);
    // total row sum = sum of the two halves
    s_rowsum[half * 128 + r] = l_run;
    __syncwarp();
    if (lane == 0) mbar_arrive(x_bar);
    ok = ok && mbar_wait(x_bar, ntiles & 1, abort_flag, p.status);
    const float l_tot = l_run + s_rowsum[(half ^ 1) * 128 + r];
    if (ok && row_valid) {
      const float inv = l_tot > 0.f ? (DROP ? p.drop.keep_scale : 1.f) / l_tot : 0.f;
      __nv_bfloat16* orow = p.O + (((long long)b * p.Sq + i) * p.Hq + h) * HDIM + half * (HDIM / 2);
#pragma unroll
      for (int c = 0; c < HDIM / 2; c += 8) {
        uint4 v;
        v.x = pack_bf16x2(o_acc[c] * inv, o_acc[c + 1] * inv);
        v.y = pack_bf16x2(o_acc[c + 2] * inv, o_acc[c + 3] * inv);
        v.z = pack_bf16x2(o_acc[c + 4] * inv, o_acc[c + 5] * inv);
        v.w = pack_bf16x2(o_acc[c + 6] * inv, o_acc[c + 7] * inv);
        *reinterpret_cast<uint4*>(orow + c) = v;
      }
      if (half == 0)
        p.lse[((long long)b * p.Hq + h) * p.Sq + i] =
            l_tot > 0.f ? (m_run * p.scale_log2 + log2f(l_tot)) * 0.6931471805599453f : -INFINITY;
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

// q: rows = B*Sq tokens with pitch q_stride elements, head h at columns [h*128, h*128+128);
// k, v likewise with B*Sk rows. O: [B, Sq, Hq, head_dim] contiguous bf16; lse: [B, Hq, Sq] fp32.
// row_lo / row_hi: optional int32 [B, Sq] key intervals (see file header).
template <bool DROP, bool BIAS, int HDIM>
static int fwd_variant(dim3 grid, cudaStream_t st, const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV,
                       const FwdParams& p) {
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(flash_fwd_kernel<DROP, BIAS, HDIM>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             SmemLayout::TOTAL) != cudaSuccess)
      return -4;
    attr_set = true;
  }
  flash_fwd_kernel<DROP, BIAS, HDIM><<<grid, THREADS, SmemLayout::TOTAL, st>>>(tmQ, tmK, tmV, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

static int flash_fwd_launch(const void* q, const void* k, const void* v, void* o, float* lse, const int* row_lo,
                            const int* row_hi, int B, int Sq, int Sk, int Hq, int Hkv, long long q_stride,
                            long long k_stride, long long v_stride, int causal, float softmax_scale, void* stream,
                            int* status, DropParams drop, BiasParams bias = BiasParams{nullptr, 0, 0, 0},
                            int head_dim = 128) {
  if (B <= 0 || Sq <= 0 || Sk <= 0) return 0;
  if (head_dim != 128 && head_dim != 64) return -1;
  const int HDv = head_dim;
  if (Hq % Hkv) return -1;
  if ((q_stride | k_stride | v_stride) & 7) return -1;
  CUtensorMap tmQ, tmK, tmV;
  if (!make_tmap_2d(&tmQ, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)B * Sq, (uint64_t)Hq * HDv, q_stride, BQ,
                    64, CU_TENSOR_MAP_SWIZZLE_128B))
    return -2;
  if (!make_tmap_2d(&tmK, k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)B * Sk, (uint64_t)Hkv * HDv, k_stride,
                    BKV, 64, CU_TENSOR_MAP_SWIZZLE_128B))
    return -2;
  if (!make_tmap_2d(&tmV, v, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)B * Sk, (uint64_t)Hkv * HDv, v_stride,
                    BKV, 64, CU_TENSOR_MAP_SWIZZLE_128B))
    return -2;
  FwdParams p;
  p.O = (__nv_bfloat16*)o; p.lse = lse; p.row_lo = row_lo; p.row_hi = row_hi;
  p.B = B; p.Sq = Sq; p.Sk = Sk; p.Hq = Hq; p.Hkv = Hkv; p.causal = causal;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.status = status;
  p.drop = drop;
  p.bias = bias;
  p.inv_scale = 1.f / softmax_scale;
  if (bias.ptr != nullptr &&
      ((Sk & 7) || ((bias.sb | bias.sh | bias.sq) & 7) || (reinterpret_cast<uintptr_t>(bias.ptr) & 15) ||
       !(softmax_scale > 0.f)))
    return -1;
  dim3 grid((Sq + BQ - 1) / BQ, Hq, B);
  const cudaStream_t st = (cudaStream_t)stream;
  const bool dr = drop.thr16 != 0, bi = bias.ptr != nullptr;
#define ATB_FWD_PICK(HD_)                                                             \
  do {                                                                                \
    if (dr && bi) return fwd_variant<true, true, HD_>(grid, st, tmQ, tmK, tmV, p);     \
    if (dr) return fwd_variant<true, false, HD_>(grid, st, tmQ, tmK, tmV, p);          \
    if (bi) return fwd_variant<false, true, HD_>(grid, st, tmQ, tmK, tmV, p);          \
    return fwd_variant<false, false, HD_>(grid, st, tmQ, tmK, tmV, p);                 \
  } while (0)
  if (head_dim == 64) ATB_FWD_PICK(64);
  ATB_FWD_PICK(128);
#undef ATB_FWD_PICK
}

extern "C" int atb_flash_fwd(const void* q, const void* k, const void* v, void* o, float* lse, const int* row_lo,
                             const int* row_hi, int B, int Sq, int Sk, int Hq, int Hkv, long long q_stride,
                             long long k_stride, long long v_stride, int causal, float softmax_scale, void* stream,
                             int* status) {
  return flash_fwd_launch(q, k, v, o, lse, row_lo, row_hi, B, Sq, Sk, Hq, Hkv, q_stride, k_stride, v_stride, causal,
                          softmax_scale, stream, status, DropParams{0u, 0u, 0u, 1.f});
}

// The same with attention dropout: probability thr16 / 65536 (0 < thr16 < 65536), mask defined by the seed pair
// (common.cuh: drop_row_key / drop_pair_bits); the backward must be given the same three numbers.
extern "C" int atb_flash_fwd_dropout(const void* q, const void* k, const void* v, void* o, float* lse,
                                     const int* row_lo, const int* row_hi, int B, int Sq, int Sk, int Hq, int Hkv,
                                     long long q_stride, long long k_stride, long long v_stride, int causal,
                                     float softmax_scale, void* stream, int* status, unsigned thr16,
                                     unsigned seed_lo, unsigned seed_hi) {
  if (thr16 == 0 || thr16 >= 65536u) return -1;
  return flash_fwd_launch(q, k, v, o, lse, row_lo, row_hi, B, Sq, Sk, Hq, Hkv, q_stride, k_stride, v_stride, causal,
                          softmax_scale, stream, status,
                          DropParams{thr16, seed_lo, seed_hi, 65536.f / (float)(65536u - thr16)});
}

// With an additive bias on the scaled scores (see BiasParams in common.cuh) and, if thr16 != 0, dropout.
extern "C" int atb_flash_fwd_bias(const void* q, const void* k, const void* v, void* o, float* lse, const int* row_lo,
                                  const int* row_hi, int B, int Sq, int Sk, int Hq, int Hkv, long long q_stride,
                                  long long k_stride, long long v_stride, int causal, float softmax_scale,
                                  void* stream, int* status, unsigned thr16, unsigned seed_lo, unsigned seed_hi,
                                  const void* bias, long long bias_sb, long long bias_sh, long long bias_sq) {
  if (thr16 >= 65536u || bias == nullptr) return -1;
  const DropParams drop = thr16 ? DropParams{thr16, seed_lo, seed_hi, 65536.f / (float)(65536u - thr16)}
                                : DropParams{0u, 0u, 0u, 1.f};
  return flash_fwd_launch(q, k, v, o, lse, row_lo, row_hi, B, Sq, Sk, Hq, Hkv, q_stride, k_stride, v_stride, causal,
                          softmax_scale, stream, status, drop,
                          BiasParams{(const __nv_bfloat16*)bias, bias_sb, bias_sh, bias_sq});
}

// The general entry point: head dim 128 or 64, optional dropout (thr16 != 0) and additive bias (bias != null).
extern "C" int atb_flash_fwd_ex(const void* q, const void* k, const void* v, void* o, float* lse, const int* row_lo,
                                const int* row_hi, int B, int Sq, int Sk, int Hq, int Hkv, long long q_stride,
                                long long k_stride, long long v_stride, int causal, float softmax_scale, void* stream,
                                int* status, unsigned thr16, unsigned seed_lo, unsigned seed_hi, const void* bias,
                                long long bias_sb, long long bias_sh, long long bias_sq, int head_dim) {
  if (thr16 >= 65536u) return -1;
  const DropParams drop = thr16 ? DropParams{thr16, seed_lo, seed_hi, 65536.f / (float)(65536u - thr16)}
                                : DropParams{0u, 0u, 0u, 1.f};
  return flash_fwd_launch(q, k, v, o, lse, row_lo, row_hi, B, Sq, Sk, Hq, Hkv, q_stride, k_stride, v_stride, causal,
                          softmax_scale, stream, status, drop,
                          BiasParams{(const __nv_bfloat16*)bias, bias_sb, bias_sh, bias_sq}, head_dim);
}
