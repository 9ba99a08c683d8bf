// Rotary position embedding, SwiGLU and small fused elementwise kernels for sm_100a.
//
// All are bandwidth-bound: 16-byte vector accesses, one read and one write per element.
// RoPE works in place on the q and k heads of a fused [tokens, (hq + 2*hkv) * d] projection
// output; SwiGLU reads the fused [tokens, 2*F] gate|up output of one GEMM.
//
// Counterparts in the reference: atorch/kernels/triton_jit/rope.py:4-10 and swiglu.py:4-11
// (wrappers around liger Triton kernels), atorch/kernels/triton_jit/bias_gather_add.py:13-160.
#include "common.cuh"

namespace {
using namespace atb;

// x: [T, row_stride] bf16; heads 0..nheads-1 of width D starting at column 0 are rotated:
//   out[..., :D/2] = x1*cos - x2*sin ; out[..., D/2:] = x2*cos + x1*sin   (rotate_half form)
// cos/sin: fp32 [S, D/2]; position of token t is pos[t] if pos != nullptr else t % S.
// sign = +1 forward, -1 backward (the transpose of a rotation is the rotation by -theta).
// When `src` differs from `x` the result is written to `x` from `src` (out of place) and the columns after the
// rotated heads (`tail8` 16-byte vectors per row, e.g. the v heads) are copied through unchanged.
__global__ void rope_kernel(__nv_bfloat16* x, const __nv_bfloat16* src,
                            const float* __restrict__ cosT, const float* __restrict__ sinT,
                            const int* __restrict__ pos, long long T, int S, int nheads, int D, long long row_stride,
                            long long src_stride, int tail8, float sign) {
  const int half = D >> 1;
  const int vec_per_head = half >> 3;  // 8 bf16 per 16-byte vector
  const long long total = T * (long long)nheads * vec_per_head;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int v = (int)(i % vec_per_head);
    const long long th = i / vec_per_head;
    const int h = (int)(th % nheads);
    const long long t = th / nheads;
    const int p = pos ? pos[t] : (int)(t % S);
    __nv_bfloat16* base = x + t * row_stride + (long long)h * D + v * 8;
    const __nv_bfloat16* sbase = src + t * src_stride + (long long)h * D + v * 8;
    uint4 a = *reinterpret_cast<const uint4*>(sbase);
    uint4 b = *reinterpret_cast<const uint4*>(sbase + half);
    const float4* c4 = reinterpret_cast<const float4*>(cosT + (long long)p * half + v * 8);
    const float4* s4 = reinterpret_cast<const float4*>(sinT + (long long)p * half + v * 8);
    float4 c0 = c4[0], c1 = c4[1], s0 = s4[0], s1 = s4[1];
    float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    uint32_t* au = reinterpret_cast<uint32_t*>(&a);
    uint32_t* bu = reinterpret_cast<uint32_t*>(&b);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 x1 = unpack_bf16x2(au[j]), x2 = unpack_bf16x2(bu[j]);
      float s_lo = sn[2 * j] * sign, s_hi = sn[2 * j + 1] * sign;
      float o1x = x1.x * cs[2 * j] - x2.x * s_lo, o1y = x1.y * cs[2 * j + 1] - x2.y * s_hi;
      float o2x = x2.x * cs[2 * j] + x1.x * s_lo, o2y = x2.y * cs[2 * j + 1] + x1.y * s_hi;
      au[j] = pack_bf16x2(o1x, o1y);
      bu[j] = pack_bf16x2(o2x, o2y);
    }
    *reinterpret_cast<uint4*>(base) = a;
    *reinterpret_cast<uint4*>(base + half) = b;
  }
  if (tail8 > 0 && src != x) {
    const long long ttotal = T * tail8;
    const long long off = (long long)nheads * D;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < ttotal;
         i += (long long)gridDim.x * blockDim.x) {
      const long long t = i / tail8;
      const int c = (int)(i - t * tail8) * 8;
      *reinterpret_cast<uint4*>(x + t * row_stride + off + c) =
          *reinterpret_cast<const uint4*>(src + t * src_stride + off + c);
    }
  }
}

// out[t, f] = silu(gu[t, f]) * gu[t, F + f]
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, long long T,
                                  int F, long long gu_stride, long long out_stride) {
  const int vpr = F >> 3;
  const long long total = T * vpr;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / vpr;
    const int v = (int)(i - t * vpr);
    uint4 g = *reinterpret_cast<const uint4*>(gu + t * gu_stride + v * 8);
    uint4 u = *reinterpret_cast<const uint4*>(gu + t * gu_stride + F + v * 8);
    uint4 o;
    const uint32_t* gp = reinterpret_cast<const uint32_t*>(&g);
    const uint32_t* up = reinterpret_cast<const uint32_t*>(&u);
    uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 a = unpack_bf16x2(gp[j]), b = unpack_bf16x2(up[j]);
      float ox = a.x / (1.f + __expf(-a.x)) * b.x;
      float oy = a.y / (1.f + __expf(-a.y)) * b.y;
      op[j] = pack_bf16x2(ox, oy);
    }
    *reinterpret_cast<uint4*>(out + t * out_stride + v * 8) = o;
  }
}

// dgu[t, f] = dout * up * (sig + gate*sig*(1-sig)) ; dgu[t, F+f] = dout * silu(gate)
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gu, const __nv_bfloat16* __restrict__ dout,
                                  __nv_bfloat16* __restrict__ dgu, long long T, int F, long long gu_stride,
                                  long long dout_stride) {
  const int vpr = F >> 3;
  const long long total = T * vpr;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / vpr;
    const int v = (int)(i - t * vpr);
    uint4 g = *reinterpret_cast<const uint4*>(gu + t * gu_stride + v * 8);
    uint4 u = *reinterpret_cast<const uint4*>(gu + t * gu_stride + F + v * 8);
    uint4 d = *reinterpret_cast<const uint4*>(dout + t * dout_stride + v * 8);
    uint4 og, ou;
    const uint32_t* gp = reinterpret_cast<const uint32_t*>(&g);
    const uint32_t* up = reinterpret_cast<const uint32_t*>(&u);
    const uint32_t* dp = reinterpret_cast<const uint32_t*>(&d);
    uint32_t* ogp = reinterpret_cast<uint32_t*>(&og);
    uint32_t* oup = reinterpret_cast<uint32_t*>(&ou);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 a = unpack_bf16x2(gp[j]), b = unpack_bf16x2(up[j]), dd = unpack_bf16x2(dp[j]);
      float sx = 1.f / (1.f + __expf(-a.x)), sy = 1.f / (1.f + __expf(-a.y));
      float dgx = dd.x * b.x * (sx + a.x * sx * (1.f - sx));
      float dgy = dd.y * b.y * (sy + a.y * sy * (1.f - sy));
      float dux = dd.x * a.x * sx, duy = dd.y * a.y * sy;
      ogp[j] = pack_bf16x2(dgx, dgy);
      oup[j] = pack_bf16x2(dux, duy);
    }
    *reinterpret_cast<uint4*>(dgu + t * gu_stride + v * 8) = og;
    *reinterpret_cast<uint4*>(dgu + t * gu_stride + F + v * 8) = ou;
  }
}

// out[t, :] = inp[t, :] + bias[expert[t], :]   (MoE per-expert bias)
__global__ void bias_gather_add_kernel(const __nv_bfloat16* __restrict__ inp, const __nv_bfloat16* __restrict__ bias,
                                       const int* __restrict__ expert, __nv_bfloat16* __restrict__ out, long long T,
                                       int H) {
  const int vpr = H >> 3;
  const long long total = T * vpr;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / vpr;
    const int v = (int)(i - t * vpr);
    const int e = expert[t];
    uint4 a = *reinterpret_cast<const uint4*>(inp + t * H + v * 8);
    uint4 b = *reinterpret_cast<const uint4*>(bias + (long long)e * H + v * 8);
    uint32_t* ap = reinterpret_cast<uint32_t*>(&a);
    const uint32_t* bp = reinterpret_cast<const uint32_t*>(&b);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 x = unpack_bf16x2(ap[j]), y = unpack_bf16x2(bp[j]);
      ap[j] = pack_bf16x2(x.x + y.x, x.y + y.y);
    }
    *reinterpret_cast<uint4*>(out + t * H + v * 8) = a;
  }
}

// y = a + b (bf16), 8 elements per thread
__global__ void add_bf16_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                                __nv_bfloat16* __restrict__ y, long long n8) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8;
       i += (long long)gridDim.x * blockDim.x) {
    uint4 x = reinterpret_cast<const uint4*>(a)[i], z = reinterpret_cast<const uint4*>(b)[i];
    uint32_t* xp = reinterpret_cast<uint32_t*>(&x);
    const uint32_t* zp = reinterpret_cast<const uint32_t*>(&z);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 p = unpack_bf16x2(xp[j]), q = unpack_bf16x2(zp[j]);
      xp[j] = pack_bf16x2(p.x + q.x, p.y + q.y);
    }
    reinterpret_cast<uint4*>(y)[i] = x;
  }
}

inline int grid_for(long long work, int threads) {
  long long g = (work + threads - 1) / threads;
  long long cap = 148LL * 16;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}
}  // namespace

// `src` == nullptr or == x: in place. Otherwise x (pitch row_stride) = rope(src (pitch src_stride)) and the
// `tail_cols` columns after the rotated heads are copied unchanged.
extern "C" int atb_rope(void* x, const void* src, const float* cosT, const float* sinT, const int* pos, long long T,
                        int S, int nheads, int D, long long row_stride, long long src_stride, int tail_cols,
                        int backward, void* stream) {
  if (T <= 0 || nheads <= 0) return 0;
  if ((D & 15) || (row_stride & 7) || (src_stride & 7) || (tail_cols & 7)) return -1;
  const long long total = T * (long long)nheads * (D >> 4);
  const __nv_bfloat16* s = src ? (const __nv_bfloat16*)src : (const __nv_bfloat16*)x;
  rope_kernel<<<grid_for(total, 256), 256, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)x, s, cosT, sinT, pos, T, S, nheads,
                                                                      D, row_stride, src ? src_stride : row_stride,
                                                                      tail_cols >> 3, backward ? -1.f : 1.f);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
extern "C" int atb_swiglu_fwd(const void* gu, void* out, long long T, int F, long long gu_stride, long long out_stride,
                              void* stream) {
  if (T <= 0) return 0;
  if ((F & 7) || (gu_stride & 7) || (out_stride & 7)) return -1;
  swiglu_fwd_kernel<<<grid_for(T * (F >> 3), 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, T, F, gu_stride, out_stride);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
extern "C" int atb_swiglu_bwd(const void* gu, const void* dout, void* dgu, long long T, int F, long long gu_stride,
                              long long dout_stride, void* stream) {
  if (T <= 0) return 0;
  if ((F & 7) || (gu_stride & 7) || (dout_stride & 7)) return -1;
  swiglu_bwd_kernel<<<grid_for(T * (F >> 3), 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)gu, (const __nv_bfloat16*)dout, (__nv_bfloat16*)dgu, T, F, gu_stride, dout_stride);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
extern "C" int atb_bias_gather_add(const void* inp, const void* bias, const int* expert, void* out, long long T, int H,
                                   void* stream) {
  if (T <= 0) return 0;
  if (H & 7) return -1;
  bias_gather_add_kernel<<<grid_for(T * (H >> 3), 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)inp, (const __nv_bfloat16*)bias, expert, (__nv_bfloat16*)out, T, H);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
extern "C" int atb_add_bf16(const void* a, const void* b, void* y, long long n, void* stream) {
  if (n <= 0) return 0;
  if (n & 7) return -1;
  add_bf16_kernel<<<grid_for(n >> 3, 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)a, (const __nv_bfloat16*)b, (__nv_bfloat16*)y, n >> 3);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
