// Block-scaled FP8 (e4m3) for sm_100a: quantisers and the scaled GEMM.
//
// Scales are stored as inverse scales: x ~= q * s with s = max(amax, eps) / 448 (optionally
// rounded up to a power of two), as in the reference's Triton kernels.
//   tile  quantisation: one scale per 1 x 128 strip along the reduction dim   (activations, grads)
//   block quantisation: one scale per 128 x 128 block                         (weights)
// Both come with a *transposed-output* form (quantise X, emit X^T quantised along the new
// reduction dim), which is what the dgrad / wgrad products of a linear layer consume.
//
// GEMM: C[M,N] (+)= sum_kb (A_q[:, kb] B_q[:, kb]^T) * a_s[m, kb] * b_s[n | n/128, kb], fp32 accumulate.
// Each 128-wide K block is one tcgen05.mma (kind::f8f6f4, 4 x K=32) into a fresh TMEM accumulator
// (two buffers, ping-pong); the epilogue warps pull it out of tensor memory, apply the two scales
// and add it to a register accumulator (one output row per thread), while the tensor core works
// on the next K block. TMA feeds 128-byte-swizzled [128 x 128 B] tiles.
//
// Replaces the Triton kernels of atorch/modules/fp8/triton_kernel.py:21-210 (block_quant, tile_quant,
// dequant, fp8_gemm) and the kitchen/deep_gemm calls of atorch/modules/fp8/cuda_kernel.py:8-81.
#include "common.cuh"
#include <cuda_fp8.h>

namespace {
using namespace atb;

constexpr float FP8_MAX = 448.f;
constexpr float FP8_EPS = 1e-12f;

ATB_DEVICE float make_scale(float amax, int pow2) {
  float s = fmaxf(amax, FP8_EPS) / FP8_MAX;
  if (pow2) s = exp2f(ceilf(log2f(s)));
  return s;
}
ATB_DEVICE uint8_t to_e4m3(float v) {
  return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
}
ATB_DEVICE float from_e4m3(uint8_t b) {
  __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3);
  return __half2float(*reinterpret_cast<__half*>(&h));
}

// Two e4m3 bytes from two floats in one conversion instruction (low byte = first value).
ATB_DEVICE uint32_t to_e4m3x2(float a, float b) {
  return (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
}
ATB_DEVICE uint32_t to_e4m3x4(float a, float b, float c, float d) { return to_e4m3x2(a, b) | (to_e4m3x2(c, d) << 16); }

// ---------------------------------------------------------------------------------------------
// 1 x 128 tile quantisation, row-major in, row-major out; K % 128 == 0. A half-warp owns a tile: every
// lane loads 16 bytes (8 values) and stores 8; a warp iteration covers eight tiles (four per half-warp, all
// loads issued before the first reduction) so that enough bytes are in flight per SM. Output and scales are
// dense, so tile t lives at byte 128 t of q; only a pitched input needs the row of a tile.
// ---------------------------------------------------------------------------------------------
constexpr int TQ_E = 4;
__global__ void tile_quant_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q,
                                  float* __restrict__ scales, long long M, int K, long long ldx, int pow2) {
  const int tiles = K >> 7;
  const long long total = M * tiles;
  const bool dense = ldx == K;
  const int lane = threadIdx.x & 31, sub = lane & 15, hw = lane >> 4;
  const long long warp0 = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long w = warp0 * (2 * TQ_E); w < total; w += nwarps * (2 * TQ_E)) {
    uint4 u[TQ_E];
#pragma unroll
    for (int e = 0; e < TQ_E; ++e) {
      const long long tix = w + e * 2 + hw;
      u[e] = make_uint4(0u, 0u, 0u, 0u);
      if (tix < total) {
        long long off = tix * 128;
        if (!dense) {
          const long long row = tix / tiles;
          off = row * ldx + (tix - row * tiles) * 128;
        }
        u[e] = *reinterpret_cast<const uint4*>(x + off + sub * 8);
      }
    }
#pragma unroll
    for (int e = 0; e < TQ_E; ++e) {
      const long long tix = w + e * 2 + hw;
      const float2 a = unpack_bf16x2(u[e].x), b = unpack_bf16x2(u[e].y), c = unpack_bf16x2(u[e].z), d = unpack_bf16x2(u[e].w);
      float amax = fmaxf(fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y))),
                         fmaxf(fmaxf(fabsf(c.x), fabsf(c.y)), fmaxf(fabsf(d.x), fabsf(d.y))));
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));   // within the half-warp
      if (tix < total) {
        const float s = make_scale(amax, pow2);
        const float inv = 1.f / s;
        uint2 o;
        o.x = to_e4m3x4(a.x * inv, a.y * inv, b.x * inv, b.y * inv);
        o.y = to_e4m3x4(c.x * inv, c.y * inv, d.x * inv, d.y * inv);
        *reinterpret_cast<uint2*>(q + tix * 128 + sub * 8) = o;
        if (sub == 0) scales[tix] = s;
      }
    }
  }
}

// Transposed form: x [M, K] -> q_t [K, M] quantised in strips of 128 along M; scales_t [K, M/128].
// One CTA per [128 (M) x 64 (K)] tile; M % 128 == 0, K % 64 == 0. Four threads per output row; thread `part`
// writes bytes [16 part, 16 part + 16) and [64 + 16 part, ...) of the row's 128, so that the four stores of a
// row are one contiguous 64-byte piece each.
__global__ void __launch_bounds__(256)
tile_quant_t_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ qt, float* __restrict__ scales_t,
                    long long M, int K, long long ldx, int pow2) {
  __shared__ float tile[64][129];
  const long long m0 = (long long)blockIdx.y * 128;
  const int k0 = blockIdx.x * 64;
  for (int i = threadIdx.x; i < 128 * 8; i += 256) {  // 128 rows x 8 chunks of 8 bf16 (16 bytes)
    const int r = i >> 3, c8 = i & 7;
    const uint4 u = *reinterpret_cast<const uint4*>(x + (m0 + r) * ldx + k0 + c8 * 8);
    const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
    float* col = &tile[c8 * 8][r];
    col[0] = a.x; col[129] = a.y; col[2 * 129] = b.x; col[3 * 129] = b.y;
    col[4 * 129] = c.x; col[5 * 129] = c.y; col[6 * 129] = d.x; col[7 * 129] = d.y;
  }
  __syncthreads();
  const int k = threadIdx.x >> 2, part = threadIdx.x & 3;
  float v[32];
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    v[j] = tile[k][part * 16 + j];
    v[16 + j] = tile[k][64 + part * 16 + j];
    amax = fmaxf(amax, fmaxf(fabsf(v[j]), fabsf(v[16 + j])));
  }
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  const float s = make_scale(amax, pow2);
  const float inv = 1.f / s;
  uint8_t* dst = qt + (long long)(k0 + k) * M + m0;
#pragma unroll
  for (int hlf = 0; hlf < 2; ++hlf) {
    const float* w = v + hlf * 16;
    uint4 o;
    o.x = to_e4m3x4(w[0] * inv, w[1] * inv, w[2] * inv, w[3] * inv);
    o.y = to_e4m3x4(w[4] * inv, w[5] * inv, w[6] * inv, w[7] * inv);
    o.z = to_e4m3x4(w[8] * inv, w[9] * inv, w[10] * inv, w[11] * inv);
    o.w = to_e4m3x4(w[12] * inv, w[13] * inv, w[14] * inv, w[15] * inv);
    *reinterpret_cast<uint4*>(dst + hlf * 64 + part * 16) = o;
  }
  if (part == 0) scales_t[(long long)(k0 + k) * (M >> 7) + blockIdx.y] = s;
}

// 128 x 128 block quantisation of w [N, K]; optional transposed copy q_t [K, N] (same scales, index
// swapped by the caller). One CTA per block.
__global__ void __launch_bounds__(256)
block_quant_kernel(const __nv_bfloat16* __restrict__ w, uint8_t* __restrict__ q, uint8_t* __restrict__ qt,
                   float* __restrict__ scales, int N, int K, long long ldw, int pow2) {
  __shared__ float red[33];
  __shared__ uint8_t tq[128][132];
  const int n0 = blockIdx.y * 128, k0 = blockIdx.x * 128;
  float v[64];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 32; ++i) {  // thread handles pairs: 128 x 64 pairs / 256 threads = 32
    const int idx = threadIdx.x + i * 256;
    const int r = idx >> 6, c2 = idx & 63;
    const float2 p = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(w + (long long)(n0 + r) * ldw + k0 + c2 * 2));
    v[2 * i] = p.x;
    v[2 * i + 1] = p.y;
    amax = fmaxf(amax, fmaxf(fabsf(p.x), fabsf(p.y)));
  }
  amax = block_max(amax, red);
  const float s = make_scale(amax, pow2);
  const float inv = 1.f / s;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const int idx = threadIdx.x + i * 256;
    const int r = idx >> 6, c2 = idx & 63;
    const uint8_t a = to_e4m3(v[2 * i] * inv), b = to_e4m3(v[2 * i + 1] * inv);
    *reinterpret_cast<uint16_t*>(q + (long long)(n0 + r) * K + k0 + c2 * 2) = (uint16_t)(a | (b << 8));
    if (qt) {
      tq[c2 * 2][r] = a;
      tq[c2 * 2 + 1][r] = b;
    }
  }
  if (threadIdx.x == 0) scales[(long long)blockIdx.y * (K >> 7) + blockIdx.x] = s;
  if (qt) {
    __syncthreads();
    for (int i = threadIdx.x; i < 128 * 32; i += 256) {
      const int kk = i >> 5, c4 = i & 31;
      const uint32_t o = tq[kk][c4 * 4] | (tq[kk][c4 * 4 + 1] << 8) | (tq[kk][c4 * 4 + 2] << 16) |
                         ((uint32_t)tq[kk][c4 * 4 + 3] << 24);
      *reinterpret_cast<uint32_t*>(qt + (long long)(k0 + kk) * N + n0 + c4 * 4) = o;
    }
  }
}

// out[r, c] = q[r, c] * scale(r, c): tile mode: scales[r, c/128]; block mode: scales[r/128, c/128]
__global__ void dequant_kernel(const uint8_t* __restrict__ q, const float* __restrict__ scales,
                               __nv_bfloat16* __restrict__ out, long long R, int C, int block_mode) {
  const int tiles = C >> 7;
  const long long total = R * (C >> 2);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / (C >> 2);
    const int c = (int)(i - r * (C >> 2)) * 4;
    const float s = scales[(block_mode ? (r >> 7) : r) * tiles + (c >> 7)];
    const uint32_t u = *reinterpret_cast<const uint32_t*>(q + r * C + c);
    uint2 o;
    o.x = pack_bf16x2(from_e4m3(u & 0xff) * s, from_e4m3((u >> 8) & 0xff) * s);
    o.y = pack_bf16x2(from_e4m3((u >> 16) & 0xff) * s, from_e4m3(u >> 24) * s);
    *reinterpret_cast<uint2*>(out + r * C + c) = o;
  }
}

// ---------------------------------------------------------------------------------------------
// scaled GEMM
// ---------------------------------------------------------------------------------------------
constexpr int GBM = 128, GBN = 128, GBK = 128, GST = 6;
constexpr int G_TILE = 128 * 128;  // bytes per operand tile
constexpr int G_BAR_OFF = GST * 2 * G_TILE;
constexpr int G_SMEM = G_BAR_OFF + (2 * GST + 4) * 8 + 16 + 1024;

struct ScaledEpi {
  void* C;
  long long ldc;
  const float* a_s;  // [M, KB]
  const float* b_s;  // block mode: [N/128, KB]; row mode: [N, KB]
  int b_row_mode, out_fp32, accumulate;
};

__global__ void __launch_bounds__(192, 1)
fp8_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, ScaledEpi ep, int M,
                int N, int K, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + GST * G_TILE;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + G_BAR_OFF);
  uint64_t* empty = full + GST;
  uint64_t* tfull = empty + GST;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (status != nullptr && *reinterpret_cast<volatile int*>(status) != 0) return;
  const int tiles_m = (M + GBM - 1) / GBM, tiles_n = (N + GBN - 1) / GBN;
  const int num_tiles = tiles_m * tiles_n;
  const int KB = K / GBK;
  if (threadIdx.x == 0) {
    for (int i = 0; i < GST; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
    mbar_init(&tfull[0], 1); mbar_init(&tfull[1], 1);
    mbar_init(&tempty[0], 4); mbar_init(&tempty[1], 4);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc<1>(tmem_slot, 256); tmem_relinquish<1>(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
        const int m0 = (tile % tiles_m) * GBM, n0 = (tile / tiles_m) * GBN;
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const int s = it % GST;
          if (!mbar_wait(&empty[s], ((it / GST) & 1) ^ 1, abort_flag, status)) goto prod_done;
          mbar_expect_tx(&full[s], 2 * G_TILE);
          tma_load_2d(sA + s * G_TILE, &tmA, &full[s], kb * GBK, m0);
          tma_load_2d(sB + s * G_TILE, &tmB, &full[s], kb * GBK, n0);
        }
      }
    }
  prod_done:;
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(GBM, GBN, 0, 0, false, false);
      uint32_t it = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const int s = it % GST, buf = it & 1;
          if (!mbar_wait(&tempty[buf], ((it >> 1) & 1) ^ 1, abort_flag, status)) goto mma_done;
          if (!mbar_wait(&full[s], (it / GST) & 1, abort_flag, status)) goto mma_done;
          tc_fence_after();
          const uint32_t a_addr = smem_u32(sA + s * G_TILE), b_addr = smem_u32(sB + s * G_TILE);
#pragma unroll
          for (int k = 0; k < GBK / 32; ++k)
            umma_f8(tmem_base + buf * GBN, umma_desc_sw128(a_addr + k * 32, 16, 1024),
                    umma_desc_sw128(b_addr + k * 32, 16, 1024), idesc, k != 0);
          umma_commit(&empty[s]);
          umma_commit(&tfull[buf]);
        }
      }
    }
  mma_done:;
  } else {
    const int q = warp & 3;
    uint32_t it = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      const int m0 = (tile % tiles_m) * GBM, n0 = (tile / tiles_m) * GBN;
      const int row = m0 + q * 32 + lane;
      const bool row_ok = row < M;
      float acc[GBN];
#pragma unroll
      for (int c = 0; c < GBN; ++c) acc[c] = 0.f;
      bool ok = true;
      for (int kb = 0; kb < KB; ++kb, ++it) {
        const int buf = it & 1;
        if (!__all_sync(0xffffffffu, mbar_wait(&tfull[buf], (it >> 1) & 1, abort_flag, status))) { ok = false; break; }
        tc_fence_after();
        const float as = row_ok ? ep.a_s[(long long)row * KB + kb] : 0.f;
        const float bs_blk = ep.b_row_mode ? 0.f : ep.b_s[(long long)(n0 >> 7) * KB + kb];
        const uint32_t t_addr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * GBN;
#pragma unroll
        for (int cc = 0; cc < GBN / 32; ++cc) {
          uint32_t r[32];
          tmem_ld_32x32(t_addr + cc * 32, r);
          tmem_ld_wait();
          if (!ep.b_row_mode) {
            const float sc = as * bs_blk;
#pragma unroll
            for (int c = 0; c < 32; ++c) acc[cc * 32 + c] = fmaf(__uint_as_float(r[c]), sc, acc[cc * 32 + c]);
          } else {
#pragma unroll
            for (int c = 0; c < 32; ++c) {
              const int col = n0 + cc * 32 + c;
              const float bs = col < N ? __ldg(ep.b_s + (long long)col * KB + kb) : 0.f;
              acc[cc * 32 + c] = fmaf(__uint_as_float(r[c]), as * bs, acc[cc * 32 + c]);
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty[buf]);
      }
      if (!ok) break;
      if (row_ok) {
        if (ep.out_fp32) {
          float* crow = reinterpret_cast<float*>(ep.C) + (long long)row * ep.ldc + n0;
#pragma unroll
          for (int c = 0; c < GBN; c += 4) {
            if (n0 + c < N) {
              float4 o = make_float4(acc[c], acc[c + 1], acc[c + 2], acc[c + 3]);
              if (ep.accumulate) {
                const float4 old = *reinterpret_cast<const float4*>(crow + c);
                o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
              }
              *reinterpret_cast<float4*>(crow + c) = o;
            }
          }
        } else {
          __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(ep.C) + (long long)row * ep.ldc + n0;
#pragma unroll
          for (int c = 0; c < GBN; c += 8) {
            if (n0 + c < N) {
              uint4 o;
              o.x = pack_bf16x2(acc[c], acc[c + 1]);
              o.y = pack_bf16x2(acc[c + 2], acc[c + 3]);
              o.z = pack_bf16x2(acc[c + 4], acc[c + 5]);
              o.w = pack_bf16x2(acc[c + 6], acc[c + 7]);
              *reinterpret_cast<uint4*>(crow + c) = o;
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  if (warp == 1) { tc_fence_after(); tmem_dealloc<1>(tmem_base, 256); }
}

inline int grid_cap(long long work, int threads, int cap_mult) {
  long long g = (work + threads - 1) / threads;
  const long long cap = 148LL * cap_mult;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}
}  // namespace

extern "C" int atb_fp8_tile_quant(const void* x, void* q, float* scales, long long M, int K, long long ldx, int pow2,
                                  void* stream) {
  if (M <= 0) return 0;
  if ((K & 127) || (ldx & 7) || ((uintptr_t)x & 15) || ((uintptr_t)q & 7)) return -1;   // 16-byte loads, 8-byte stores
  tile_quant_kernel<<<grid_cap(M * (K >> 7) * (16 / TQ_E), 256, 16), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, (uint8_t*)q, scales, M, K, ldx, pow2);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
extern "C" int atb_fp8_tile_quant_t(const void* x, void* qt, float* scales_t, long long M, int K, long long ldx,
                                    int pow2, void* stream) {
  if (M <= 0) return 0;
  if ((M & 127) || (K & 63) || (ldx & 7) || ((uintptr_t)x & 15) || ((uintptr_t)qt & 15)) return -1;
  dim3 grid(K / 64, (unsigned)(M / 128));
  tile_quant_t_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, (uint8_t*)qt, scales_t, M, K,
                                                             ldx, pow2);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
extern "C" int atb_fp8_block_quant(const void* w, void* q, void* qt, float* scales, int N, int K, long long ldw,
                                   int pow2, void* stream) {
  if ((N & 127) || (K & 127) || (ldw & 1)) return -1;
  dim3 grid(K / 128, N / 128);
  block_quant_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)w, (uint8_t*)q, (uint8_t*)qt,
                                                            scales, N, K, ldw, pow2);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
extern "C" int atb_fp8_dequant(const void* q, const float* scales, void* out, long long R, int C, int block_mode,
                               void* stream) {
  if (R <= 0) return 0;
  if (C & 127) return -1;
  dequant_kernel<<<grid_cap(R * (C >> 2), 256, 16), 256, 0, (cudaStream_t)stream>>>(
      (const uint8_t*)q, scales, (__nv_bfloat16*)out, R, C, block_mode);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// A_q [M, K] e4m3 (tile scales a_s [M, K/128]); B_q [N, K] e4m3 with block scales [N/128, K/128]
// (b_row_mode = 0) or per-row tile scales [N, K/128] (b_row_mode = 1). K % 128 == 0, N % 8 == 0.
extern "C" int atb_fp8_gemm(const void* Aq, const void* Bq, const float* a_s, const float* b_s, void* C, int M, int N,
                            int K, long long ldc, int b_row_mode, int out_fp32, int accumulate, void* stream,
                            int* status) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((K & 127) || (N & 7)) return -1;
  CUtensorMap tmA, tmB;
  if (!make_tmap_2d(&tmA, Aq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K, K, GBM, GBK, CU_TENSOR_MAP_SWIZZLE_128B))
    return -2;
  if (!make_tmap_2d(&tmB, Bq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, K, K, GBN, GBK, CU_TENSOR_MAP_SWIZZLE_128B))
    return -3;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(fp8_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, G_SMEM) != cudaSuccess)
      return -4;
    attr_set = true;
  }
  ScaledEpi ep{C, ldc, a_s, b_s, b_row_mode, out_fp32, accumulate};
  const int tiles = ((M + GBM - 1) / GBM) * ((N + GBN - 1) / GBN);
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = tiles < sms ? tiles : sms;
  fp8_gemm_kernel<<<grid, 192, G_SMEM, (cudaStream_t)stream>>>(tmA, tmB, ep, M, N, K, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
