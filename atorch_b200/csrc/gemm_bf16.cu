// bf16 GEMM for sm_100a: TMA -> shared memory -> tcgen05.mma -> TMEM -> epilogue.
//
//   C[M,N] (+)= alpha * A[M,K] * B[N,K]^T        (fp32 accumulation in tensor memory)
//
// Either operand may be stored K-major (reduction dim contiguous: A[M][K], B[N][K]) or
// MN-major (A stored as [K][M], B stored as [K][N]); the three combinations used by a
// linear layer are
//   forward  y  = x W^T   : A = x  (K-major),  B = W (K-major)
//   dgrad    dx = dy W    : A = dy (K-major),  B = W (MN-major, reduction over W's rows)
//   wgrad    dW = dy^T x  : A = dy (MN-major), B = x (MN-major)
// so no operand is ever transposed in memory.
//
// Structure: persistent CTAs (one per SM), 128 x BN output tile, BK = 64, STAGES-deep
// TMA ring. Warp 0 = TMA producer, warp 1 = MMA issuer (one elected thread) and TMEM
// owner, warps 2..5 = epilogue. Two TMEM accumulators (2 x BN columns) let the epilogue
// of tile i overlap the main loop of tile i+1. All waits are bounded.
//
// Plays the role of the cuBLAS calls behind nn.Linear / torch.matmul in the reference
// (atorch/modules/distributed_modules/layers.py:117-151 and every HF Llama projection).
#include "common.cuh"

namespace {

using namespace atb;

constexpr int BM = 128;
constexpr int BK = 64;

struct EpilogueParams {
  void* C;           // output, row-major, pitch ldc elements
  const void* bias;  // optional bf16 bias[N] (nullptr = none)
  long long ldc;
  float alpha;
  int out_fp32;    // 0: bf16 output, 1: fp32 output
  int accumulate;  // 1: C += result
  const void* residual;  // optional bf16 [M, N] added in the epilogue (pitch ldr); bf16 output only
  long long ldr;
};

template <int BN, int STAGES>
struct Smem {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int BAR_OFF = STAGES * (A_BYTES + B_BYTES);
  static constexpr int TOTAL = BAR_OFF + (2 * STAGES + 4) * 8 + 16 + 1024;  // + alignment slack
};

template <int BN, int STAGES, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(192, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, EpilogueParams ep,
                 int M, int N, int K, int* status) {
  using S = Smem<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * S::A_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + S::BAR_OFF);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // a wait already ran out somewhere in this stream of work: do not start, so that a failing
  // launch ends after one wait limit instead of one per wave of CTAs
  if (status != nullptr && *reinterpret_cast<volatile int*>(status) != 0) return;

  const int tiles_m = (M + BM - 1) / BM;
  const int tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (K + BK - 1) / BK;
  constexpr int BAND = 16;  // M-tiles per band: tiles running together share A and B panels in L2

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    mbar_init(&tfull[0], 1);
    mbar_init(&tfull[1], 1);
    mbar_init(&tempty[0], 4);
    mbar_init(&tempty[1], 4);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc<1>(tmem_slot, 2 * BN);
    tmem_relinquish<1>();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  auto tile_coords = [&](int tile, int& m0, int& n0) {
    const int band_tiles = BAND * tiles_n;
    const int band = tile / band_tiles;
    const int rem = tile - band * band_tiles;
    const int rows_in_band = min(BAND, tiles_m - band * BAND);
    const int tn = rem / rows_in_band;
    const int tm = band * BAND + (rem - tn * rows_in_band);
    m0 = tm * BM;
    n0 = tn * BN;
  };

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      uint32_t it = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
        int m0, n0;
        tile_coords(tile, m0, n0);
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, status)) goto producer_done;
          mbar_expect_tx(&full[s], S::A_BYTES + S::B_BYTES);
          uint8_t* a_dst = sA + s * S::A_BYTES;
          uint8_t* b_dst = sB + s * S::B_BYTES;
          if constexpr (!A_MN) {
            tma_load_2d(a_dst, &tmA, &full[s], kb * BK, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d(a_dst + j * 8192, &tmA, &full[s], m0 + j * 64, kb * BK);
          }
          if constexpr (!B_MN) {
            tma_load_2d(b_dst, &tmB, &full[s], kb * BK, n0);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_2d(b_dst + j * 8192, &tmB, &full[s], n0 + j * 64, kb * BK);
          }
        }
      }
    }
  producer_done:;
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(BM, BN, 1, 1, A_MN, B_MN);
      uint32_t it = 0;
      int local = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local) {
        const int acc = local & 1;
        const uint32_t acc_ph = (local >> 1) & 1;
        if (!mbar_wait(&tempty[acc], acc_ph ^ 1, abort_flag, status)) goto mma_done;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&full[s], ph, abort_flag, status)) goto mma_done;
          tc_fence_after();
          const uint32_t a_addr = smem_u32(sA + s * S::A_BYTES);
          const uint32_t b_addr = smem_u32(sB + s * S::B_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t adesc = A_MN ? umma_desc_sw128(a_addr + k * 2048, 8192, 1024)
                                        : umma_desc_sw128(a_addr + k * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? umma_desc_sw128(b_addr + k * 2048, 8192, 1024)
                                        : umma_desc_sw128(b_addr + k * 32, 16, 1024);
            umma_f16<1>(d_tmem, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&empty[s]);  // frees the smem slot once these MMAs have read it
        }
        umma_commit(&tfull[acc]);  // accumulator complete
      }
    }
  mma_done:;
  } else {
    // ---------------- epilogue (warps 2..5) ----------------
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    int local = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local) {
      int m0, n0;
      tile_coords(tile, m0, n0);
      const int acc = local & 1;
      const uint32_t acc_ph = (local >> 1) & 1;
      if (!__all_sync(0xffffffffu, mbar_wait(&tfull[acc], acc_ph, abort_flag, status))) break;
      tc_fence_after();
      const int row = m0 + q * 32 + lane;
      const uint32_t t_addr = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN;
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
          if (ep.out_fp32) {
            float* crow = reinterpret_cast<float*>(ep.C) + (long long)row * ep.ldc + col0;
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              if (col0 + i < N) {  // N % 8 == 0: a 4-vector is entirely in or out
                float4 o = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
                if (ep.accumulate) {
                  float4 old = *reinterpret_cast<const float4*>(crow + i);
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
                  uint4 old = *reinterpret_cast<const uint4*>(crow + i);
                  float2 o0 = unpack_bf16x2(old.x), o1 = unpack_bf16x2(old.y), o2 = unpack_bf16x2(old.z),
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
      if (lane == 0) mbar_arrive(&tempty[acc]);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // a wait ran out: give copies still in flight time to land before the CTA's memory is reused
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<1>(tmem_base, 2 * BN);
  }
}

int g_num_sms = 0;
int num_sms() {
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_num_sms <= 0) g_num_sms = 148;
  }
  return g_num_sms;
}

template <int BN, int STAGES, bool A_MN, bool B_MN>
int launch(const void* A, const void* B, const EpilogueParams& ep, int M, int N, int K, long long lda, long long ldb,
           int max_ctas, cudaStream_t stream, int* status) {
  using S = Smem<BN, STAGES>;
  CUtensorMap tmA, tmB;
  bool ok;
  if (!A_MN)
    ok = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, lda, BM, BK, CU_TENSOR_MAP_SWIZZLE_128B);
  else
    ok = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, M, lda, BK, 64, CU_TENSOR_MAP_SWIZZLE_128B);
  if (!ok) return -2;
  if (!B_MN)
    ok = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, ldb, BN, BK, CU_TENSOR_MAP_SWIZZLE_128B);
  else
    ok = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, ldb, BK, 64, CU_TENSOR_MAP_SWIZZLE_128B);
  if (!ok) return -3;
  auto kern = gemm_bf16_kernel<BN, STAGES, A_MN, B_MN>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL) != cudaSuccess) return -4;
    attr_set = true;
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  int grid = tiles < num_sms() ? tiles : num_sms();
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  kern<<<grid, 192, S::TOTAL, stream>>>(tmA, tmB, ep, M, N, K, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

}  // namespace

// C[M,N] (+)= alpha * op(A) * op(B)^T + bias.  lda/ldb/ldc are row pitches in elements of the
// arrays as stored (A: [M][K] or [K][M] if a_mn_major; B: [N][K] or [K][N] if b_mn_major).
// Requirements: 16-byte aligned bases, pitches multiples of 8 elements, N % 8 == 0.
// `status` is a device int that receives an AtbStatus code if a wait inside the kernel ran out.
// `max_ctas` > 0 caps the persistent grid (leaves SMs free for a concurrent kernel).
// Returns 0 on launch, negative on a rejected argument.
extern "C" int atb_gemm_bf16(const void* A, const void* B, void* C, const void* bias, int M, int N, int K,
                             long long lda, long long ldb, long long ldc, int a_mn_major, int b_mn_major,
                             int out_fp32, int accumulate, float alpha, int tile_n, int max_ctas,
                             const void* residual, long long ldr, void* stream, int* status) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((N & 7) || (lda & 7) || (ldb & 7) || (ldc & 3) || (!out_fp32 && (ldc & 7))) return -1;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15)
    return -1;
  if (residual != nullptr && (out_fp32 || (ldr & 7) || (reinterpret_cast<uintptr_t>(residual) & 15))) return -1;
  EpilogueParams ep{C, bias, ldc, alpha, out_fp32, accumulate, residual, ldr};
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const bool wide = (tile_n == 256) || (tile_n == 0 && N >= 256);
#define ATB_DISPATCH(BN_, ST_)                                                                              \
  do {                                                                                                      \
    if (!a_mn_major && !b_mn_major)                                                                         \
      return launch<BN_, ST_, false, false>(A, B, ep, M, N, K, lda, ldb, max_ctas, st, status);            \
    if (!a_mn_major && b_mn_major)                                                                          \
      return launch<BN_, ST_, false, true>(A, B, ep, M, N, K, lda, ldb, max_ctas, st, status);             \
    if (a_mn_major && b_mn_major)                                                                           \
      return launch<BN_, ST_, true, true>(A, B, ep, M, N, K, lda, ldb, max_ctas, st, status);              \
    return launch<BN_, ST_, true, false>(A, B, ep, M, N, K, lda, ldb, max_ctas, st, status);               \
  } while (0)
  if (wide) ATB_DISPATCH(256, 4);
  ATB_DISPATCH(128, 6);
#undef ATB_DISPATCH
}
