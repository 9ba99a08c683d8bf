// Flash attention backward, query-gradient kernel for sm_100a (head dim 128, bf16), tcgen05 + TMEM + TMA.
//
// One CTA per (128 query rows, head, batch) walks the key blocks its rows can see and keeps dQ in tensor
// memory from the first block to the last, so the query gradient needs no atomic adds, no fp32 scratch buffer
// and no conversion pass (the key/value gradients come from the key-block kernel of flash_attn_bwd.cu):
//   S  = Q K_j^T,  dP = dO V_j^T              2 x tcgen05.mma  smem x smem -> TMEM
//   P  = exp2(S c - lse),  dS = P (dP - delta) s   registers; dS written as bf16 over the dP columns
//   dQ += dS K_j                                tcgen05.mma  TMEM x smem (MN-major K) -> TMEM
// TMEM: S | dP (two buffers) | dQ = 4 x 128 columns. While the element-wise warps work on block j the tensor
// core already forms S and dP of block j+1 (S is free as soon as the warps hold it in registers, dP has a
// second buffer); dQ of block j follows when dS(j) is in place.
//
// Warp 0 = TMA producer (Q, dO once; K in three stages because a K tile serves S and, later, dQ; V in two),
// warp 1 = MMA issuer / TMEM owner, warps 2..9 = element-wise work: thread (row r, half h) owns columns
// [64h, 64h+64) of row r. The two threads of a row sit in different warps and the bf16 dS of one overwrites
// fp32 dP columns of the other, so the two warps of a lane quarter meet at a barrier between loading
// and storing (an mbarrier with a bounded wait). Masks are per-row key intervals [lo, hi) as in the forward kernel.
#include "common.cuh"

namespace {
using namespace atb;

constexpr int BQ = 128, BKV = 128, HD = 128;
constexpr int PANEL = 128 * 64 * 2;
constexpr int TILE = 2 * PANEL;
constexpr int K_STAGES = 3, V_STAGES = 2;
constexpr int N_EW = 256;
constexpr int THREADS = 64 + N_EW;

struct DqParams {
  const float* lse;    // [B, Hq, Sq]
  const float* delta;  // [B, Hq, Sq]
  __nv_bfloat16* dq;   // token-major, head h at columns [h*HD, h*HD+HD) of a row of pitch dq_stride
  long long dq_stride;
  const int* row_lo;
  const int* row_hi;
  int B, Sq, Sk, Hq, Hkv, causal;
  float scale, scale_log2;
  int* status;
};

struct SmemQ {
  static constexpr int Q_OFF = 0;
  static constexpr int DO_OFF = Q_OFF + TILE;
  static constexpr int K_OFF = DO_OFF + TILE;
  static constexpr int V_OFF = K_OFF + K_STAGES * TILE;
  static constexpr int BAR_OFF = V_OFF + V_STAGES * TILE;  // 224 KB
  static constexpr int NBARS = 1 + 2 * K_STAGES + 2 * V_STAGES + 4 + 4;
  static constexpr int TOTAL = BAR_OFF + NBARS * 8 + 64 + 1024;
};
static_assert(SmemQ::TOTAL <= 232448, "shared memory of the dQ kernel exceeds 227 KB");

__global__ void __launch_bounds__(THREADS, 1)
flash_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmdO,
                    const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, DqParams p) {
  using L = SmemQ;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + L::Q_OFF;
  uint8_t* sdO = smem + L::DO_OFF;
  uint8_t* sK = smem + L::K_OFF;
  uint8_t* sV = smem + L::V_OFF;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* qdo_full = bars;
  uint64_t* k_full = bars + 1;                 // [K_STAGES]
  uint64_t* k_empty = k_full + K_STAGES;       // [K_STAGES]  dQ(j) has read K_j
  uint64_t* v_full = k_empty + K_STAGES;       // [V_STAGES]
  uint64_t* v_empty = v_full + V_STAGES;       // [V_STAGES]  dP(j) has read V_j
  uint64_t* sdp_full = v_empty + V_STAGES;     // S(j), dP(j) are in TMEM
  uint64_t* s_free = sdp_full + 1;             // every element-wise warp holds S(j), dP(j) in registers
  uint64_t* ds_full = s_free + 1;              // dS(j) is in TMEM
  uint64_t* dq_full = ds_full + 1;             // the last dQ product has completed
  uint64_t* pair_bar = dq_full + 1;            // [4] the two warps of a lane quarter both hold S(j), dP(j)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + L::NBARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* kv_range = const_cast<int*>(reinterpret_cast<volatile int*>(tmem_slot + 2));  // [4]: t0, t1, full_lo, full_hi

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != 0) return;
  const int qb = gridDim.x - 1 - blockIdx.x;  // heaviest (last) causal blocks first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.Hq / p.Hkv);
  const int q0 = qb * BQ;
  const int shift = p.Sk - p.Sq;

  if (threadIdx.x == 0) {
    mbar_init(qdo_full, 1);
    for (int i = 0; i < K_STAGES; ++i) { mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1); }
    for (int i = 0; i < V_STAGES; ++i) { mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1); }
    mbar_init(sdp_full, 1);
    mbar_init(s_free, N_EW / 32);
    mbar_init(ds_full, N_EW / 32);
    mbar_init(dq_full, 1);
    for (int i = 0; i < 4; ++i) mbar_init(&pair_bar[i], 2);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc<1>(tmem_slot, 512);
    tmem_relinquish<1>();
  }
  if (warp == 2) {   // key range of this query block: union and intersection of the rows' intervals
    int umin = INT_MAX, umax = 0, ilo = 0, ihi = INT_MAX;
    for (int r = lane; r < BQ; r += 32) {
      const int i = q0 + r;
      if (i >= p.Sq) continue;
      int lo = p.row_lo ? p.row_lo[(long long)b * p.Sq + i] : 0;
      int hi = p.row_hi ? p.row_hi[(long long)b * p.Sq + i] : (p.causal ? i + 1 + shift : p.Sk);
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
  const int t0 = kv_range[0], n = kv_range[1] - kv_range[0];
  const int full_lo = kv_range[2], full_hi = kv_range[3];
  const long long q_row0 = (long long)b * p.Sq + q0;
  const long long k_row0 = (long long)b * p.Sk;
  const uint32_t tS = tmem_base, tdP = tmem_base + 128, tdQ = tmem_base + 384;   // dP buffer j&1 at tdP + 128*(j&1)

  if (warp == 0) {
    if (lane == 0 && n > 0) {
      tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmdO); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
      mbar_expect_tx(qdo_full, 2 * TILE);
      tma_load_2d(sQ, &tmQ, qdo_full, h * HD, (int)q_row0);
      tma_load_2d(sQ + PANEL, &tmQ, qdo_full, h * HD + 64, (int)q_row0);
      tma_load_2d(sdO, &tmdO, qdo_full, h * HD, (int)q_row0);
      tma_load_2d(sdO + PANEL, &tmdO, qdo_full, h * HD + 64, (int)q_row0);
      for (int j = 0; j < n; ++j) {
        const int ks = j % K_STAGES, vs = j % V_STAGES;
        const int krow = (int)(k_row0 + (long long)(t0 + j) * BKV);
        if (!mbar_wait(&k_empty[ks], ((j / K_STAGES) & 1) ^ 1, abort_flag, p.status)) break;
        mbar_expect_tx(&k_full[ks], TILE);
        tma_load_2d(sK + ks * TILE, &tmK, &k_full[ks], hk * HD, krow);
        tma_load_2d(sK + ks * TILE + PANEL, &tmK, &k_full[ks], hk * HD + 64, krow);
        if (!mbar_wait(&v_empty[vs], ((j / V_STAGES) & 1) ^ 1, abort_flag, p.status)) break;
        mbar_expect_tx(&v_full[vs], TILE);
        tma_load_2d(sV + vs * TILE, &tmV, &v_full[vs], hk * HD, krow);
        tma_load_2d(sV + vs * TILE + PANEL, &tmV, &v_full[vs], hk * HD + 64, krow);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n > 0) {
      constexpr uint32_t id_kk = umma_idesc(128, 128, 1, 1, false, false);
      constexpr uint32_t id_km = umma_idesc(128, 128, 1, 1, false, true);
      const uint64_t dQk = umma_desc_sw128(smem_u32(sQ), 16, 1024), dOk = umma_desc_sw128(smem_u32(sdO), 16, 1024);
      const uint64_t dKk0 = umma_desc_sw128(smem_u32(sK), 16, 1024), dKm0 = umma_desc_sw128(smem_u32(sK), PANEL, 1024);
      const uint64_t dVk0 = umma_desc_sw128(smem_u32(sV), 16, 1024);
      // S(j) = Q K_j^T and dP(j) = dO V_j^T
      auto issue_sdp = [&](int j) -> bool {
        const int ks = j % K_STAGES, vs = j % V_STAGES;
        if (!mbar_wait(&k_full[ks], (j / K_STAGES) & 1, abort_flag, p.status)) return false;
        tc_fence_after();
        const uint64_t kd = umma_desc_advance(dKk0, ks * TILE);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t off = (k >> 2) * PANEL + (k & 3) * 32;
          umma_f16<1>(tS, umma_desc_advance(dQk, off), umma_desc_advance(kd, off), id_kk, k != 0);
        }
        if (!mbar_wait(&v_full[vs], (j / V_STAGES) & 1, abort_flag, p.status)) return false;
        tc_fence_after();
        const uint64_t vd = umma_desc_advance(dVk0, vs * TILE);
        const uint32_t dst = tdP + 128 * (j & 1);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t off = (k >> 2) * PANEL + (k & 3) * 32;
          umma_f16<1>(dst, umma_desc_advance(dOk, off), umma_desc_advance(vd, off), id_kk, k != 0);
        }
        umma_commit(sdp_full);
        umma_commit(&v_empty[vs]);
        return true;
      };
      bool ok = mbar_wait(qdo_full, 0, abort_flag, p.status);
      ok = ok && issue_sdp(0);
      for (int j = 0; ok && j < n; ++j) {
        if (j + 1 < n) {
          if (!mbar_wait(s_free, j & 1, abort_flag, p.status)) break;
          tc_fence_after();
          if (!issue_sdp(j + 1)) break;
        }
        if (!mbar_wait(ds_full, j & 1, abort_flag, p.status)) break;
        tc_fence_after();
        const uint64_t km = umma_desc_advance(dKm0, (j % K_STAGES) * TILE);
        const uint32_t a = tdP + 128 * (j & 1);
#pragma unroll
        for (int k = 0; k < 8; ++k)   // dQ += dS K_j: 16 keys per step = 8 TMEM columns of packed bf16
          umma_f16_ts(tdQ, a + k * 8, umma_desc_advance(km, k * 2048), id_km, (j | k) != 0);
        umma_commit(&k_empty[j % K_STAGES]);
        if (j == n - 1) umma_commit(dq_full);
      }
    }
  } else {
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r = quarter * 32 + lane;
    const int i = q0 + r;   // global query row
    const uint32_t lane_addr = ((uint32_t)(quarter * 32) << 16);
    bool valid = i < p.Sq;
    int lo = 0, hi = 0;
    float lse2 = 0.f, delta = 0.f;
    if (valid) {
      const long long ridx = ((long long)b * p.Hq + h) * p.Sq + i;
      const float l = p.lse[ridx];
      if (l == -INFINITY) {
        valid = false;
      } else {
        lse2 = l * 1.4426950408889634f;
        delta = p.delta[ridx];
        lo = p.row_lo ? p.row_lo[(long long)b * p.Sq + i] : 0;
        hi = p.row_hi ? p.row_hi[(long long)b * p.Sq + i] : (p.causal ? i + 1 + shift : p.Sk);
        lo = max(lo, 0);
        hi = min(hi, p.Sk);
      }
    }
    const uint64_t sc2 = f2_pack(p.scale_log2, p.scale_log2), nl2 = f2_pack(-lse2, -lse2);
    const uint64_t nd2 = f2_pack(-delta, -delta), scl2 = f2_pack(p.scale, p.scale);
    bool ok = true;
    for (int j = 0; j < n; ++j) {
      const int kv0 = (t0 + j) * BKV;
      const uint32_t dp_addr = tdP + 128 * (j & 1) + lane_addr;
      if (!__all_sync(0xffffffffu, mbar_wait(sdp_full, j & 1, abort_flag, p.status))) { ok = false; break; }
      tc_fence_after();
      uint32_t s0[32], s1[32], d0[32], d1[32];
      tmem_ld_32x32(tS + lane_addr + half * 64, s0);
      tmem_ld_32x32(tS + lane_addr + half * 64 + 32, s1);
      tmem_ld_32x32(dp_addr + half * 64, d0);
      tmem_ld_32x32(dp_addr + half * 64 + 32, d1);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(s_free);
        mbar_arrive(&pair_bar[quarter]);
      }
      // both threads of every row of this lane quarter hold their S and dP before either stores dS (a bounded
      // mbarrier wait, not a named barrier, so that a warp whose partner gave up cannot wait forever)
      if (!__all_sync(0xffffffffu, mbar_wait(&pair_bar[quarter], j & 1, abort_flag, p.status))) { ok = false; break; }
      // tiles inside the intersection of the rows' intervals run without per-element tests
      const bool tile_full = (kv0 >= full_lo) && (kv0 + BKV <= full_hi);
      const int c0 = kv0 + half * 64;
      float pa[32], pb[32];   // P for keys c0 .. c0+31 and c0+32 .. c0+63
#pragma unroll
      for (int c = 0; c < 32; c += 2) {
        float a0, a1, b0, b1;
        f2_unpack(f2_fma(f2_pack_bits(s0[c], s0[c + 1]), sc2, nl2), a0, a1);
        f2_unpack(f2_fma(f2_pack_bits(s1[c], s1[c + 1]), sc2, nl2), b0, b1);
        pa[c] = fast_exp2(a0); pa[c + 1] = fast_exp2(a1);
        pb[c] = fast_exp2(b0); pb[c + 1] = fast_exp2(b1);
      }
      if (!tile_full) {   // a separate pass, so that fully visible tiles execute no interval tests at all
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          if (!valid || c0 + c < lo || c0 + c >= hi) pa[c] = 0.f;
          if (!valid || c0 + 32 + c < lo || c0 + 32 + c >= hi) pb[c] = 0.f;
        }
      }
      uint32_t ds[32];
#pragma unroll
      for (int c = 0; c < 32; c += 2) {
        float x0, x1, y0, y1;   // dS = P (dP - delta) scale
        f2_unpack(f2_mul(f2_mul(f2_pack(pa[c], pa[c + 1]), scl2), f2_add(f2_pack_bits(d0[c], d0[c + 1]), nd2)), x0, x1);
        f2_unpack(f2_mul(f2_mul(f2_pack(pb[c], pb[c + 1]), scl2), f2_add(f2_pack_bits(d1[c], d1[c + 1]), nd2)), y0, y1);
        ds[c >> 1] = pack_bf16x2(x0, x1);
        ds[16 + (c >> 1)] = pack_bf16x2(y0, y1);
      }
      // keys [64h, 64h+64) of the row as packed bf16: columns [32h, 32h+32) of the dP buffer
      tmem_st_32x32(dp_addr + half * 32, ds);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_full);
    }
    ok = __all_sync(0xffffffffu, ok);
    if (ok && n > 0) ok = __all_sync(0xffffffffu, mbar_wait(dq_full, 0, abort_flag, p.status));
    if (ok) {
      if (n > 0) tc_fence_after();
      __nv_bfloat16* row = p.dq + ((long long)b * p.Sq + i) * p.dq_stride + h * HD + half * 64;
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        uint32_t t[32];
        if (n > 0) {
          tmem_ld_32x32(tdQ + lane_addr + half * 64 + cc * 32, t);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int c = 0; c < 32; ++c) t[c] = 0u;
        }
        if (i < p.Sq) {
#pragma unroll
          for (int c = 0; c < 32; c += 8) {
            uint4 v;
            v.x = pack_bf16x2(__uint_as_float(t[c]), __uint_as_float(t[c + 1]));
            v.y = pack_bf16x2(__uint_as_float(t[c + 2]), __uint_as_float(t[c + 3]));
            v.z = pack_bf16x2(__uint_as_float(t[c + 4]), __uint_as_float(t[c + 5]));
            v.w = pack_bf16x2(__uint_as_float(t[c + 6]), __uint_as_float(t[c + 7]));
            *reinterpret_cast<uint4*>(row + cc * 32 + c) = v;
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

// dq rows of pitch dq_stride elements (head h at columns [h*128, h*128+128)); lse, delta: [B, Hq, Sq] fp32
// (delta = rowsum(dO * O), written by the pre-pass of atb_flash_bwd).
extern "C" int atb_flash_bwd_dq(const void* dout, const void* q, const void* k, const void* v, const float* lse,
                                const float* delta, void* dq, const int* row_lo, const int* row_hi, int B, int Sq,
                                int Sk, int Hq, int Hkv, long long q_stride, long long k_stride, long long v_stride,
                                long long do_stride, long long dq_stride, int causal, float softmax_scale,
                                void* stream, int* status) {
  if (B <= 0 || Sq <= 0 || Sk <= 0) return 0;
  if (Hq % Hkv) return -1;
  if ((q_stride | k_stride | v_stride | do_stride | dq_stride) & 7) return -1;
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
    if (cudaFuncSetAttribute(flash_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SmemQ::TOTAL) !=
        cudaSuccess)
      return -4;
    attr_set = true;
  }
  DqParams p;
  p.lse = lse; p.delta = delta; p.dq = (__nv_bfloat16*)dq; p.dq_stride = dq_stride;
  p.row_lo = row_lo; p.row_hi = row_hi;
  p.B = B; p.Sq = Sq; p.Sk = Sk; p.Hq = Hq; p.Hkv = Hkv; p.causal = causal;
  p.scale = softmax_scale; p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.status = status;
  dim3 grid((Sq + BQ - 1) / BQ, Hq, B);
  flash_bwd_dq_kernel<<<grid, THREADS, SmemQ::TOTAL, (cudaStream_t)stream>>>(tmQ, tmdO, tmK, tmV, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
