// Group-wise integer quantisation kernels for sm_100a (memory-bound, 16-byte accesses):
//   quantize / dequantize       int8 or packed int4, symmetric (scale) or asymmetric (scale, offset),
//                               one set of parameters per group of `group_size` consecutive elements
//   swizzle_quantize            quantise and emit groups in (pipeline, device, node)-major order so that
//                               a two-hop (intra-node, inter-node) all-to-all sends contiguous blocks
//   dequant_reduce              dequantise the chunks received from N peers, sum, requantise
//   optimizer-state packing     absmax-linear 8/16-bit and nonlinear (lookup-table) 4/8-bit codes with
//                               optional stochastic rounding (Philox counter per element)
// Conventions: symmetric  q = rint(x / s), s = absmax / qmax;  asymmetric q = rint((x - lo) / s) - 2^(b-1),
// s = (hi - lo) / (2^b - 1). 4-bit values are packed low nibble first.
// Counterparts in the reference: atorch/ops/csrc/quantization/{quantize,dequantize,swizzled_quantize,
// quant_reduce}.cu and atorch/ops/csrc/quantization_optimizer/quantization_optimizer.cu.
#include "common.cuh"

namespace {
using namespace atb;

template <typename T>
ATB_DEVICE float ldf(const T* p, long long i) { return to_f32<T>(p[i]); }

// one CTA (256 threads) per group
template <typename T>
__global__ void __launch_bounds__(256) quantize_kernel(const T* __restrict__ x, int8_t* __restrict__ q,
                                                       float* __restrict__ params, int group_size, int bits,
                                                       int asym, const int* __restrict__ group_map, int out_groups) {
  __shared__ float red[33];
  const int g = blockIdx.x;
  const T* xg = x + (long long)g * group_size;
  float lo = INFINITY, hi = -INFINITY;
  for (int i = threadIdx.x; i < group_size; i += 256) {
    const float v = ldf(xg, i);
    lo = fminf(lo, v);
    hi = fmaxf(hi, v);
  }
  hi = block_max(hi, red);
  lo = -block_max(-lo, red);
  const int qmax = (1 << (bits - 1)) - 1, half = 1 << (bits - 1);
  float s, off;
  if (asym) {
    s = (hi - lo) / (float)((1 << bits) - 1);
    off = lo;
  } else {
    s = fmaxf(fabsf(hi), fabsf(lo)) / (float)qmax;
    off = 0.f;
  }
  if (s == 0.f) s = 1.f;
  const float inv = 1.f / s;
  const int og = group_map ? group_map[g] : g;   // destination group (swizzled layouts)
  if (threadIdx.x == 0) {
    params[(long long)og * (asym ? 2 : 1)] = s;
    if (asym) params[(long long)og * 2 + 1] = off;
  }
  if (bits == 8) {
    int8_t* qg = q + (long long)og * group_size;
    for (int i = threadIdx.x; i < group_size; i += 256) {
      float r = rintf((ldf(xg, i) - off) * inv) - (asym ? half : 0);
      qg[i] = (int8_t)fminf(fmaxf(r, -half), qmax);
    }
  } else {
    int8_t* qg = q + (long long)og * (group_size / 2);
    for (int i = threadIdx.x; i < group_size / 2; i += 256) {
      float a = rintf((ldf(xg, 2 * i) - off) * inv) - (asym ? half : 0);
      float b = rintf((ldf(xg, 2 * i + 1) - off) * inv) - (asym ? half : 0);
      const int ia = (int)fminf(fmaxf(a, -half), qmax) & 0xF, ib = (int)fminf(fmaxf(b, -half), qmax) & 0xF;
      qg[i] = (int8_t)(ia | (ib << 4));
    }
  }
}

ATB_DEVICE float deq(int v, float s, float off, int asym, int half) { return asym ? (v + half) * s + off : v * s; }
ATB_DEVICE int sext4(int v) { return (v & 8) ? v - 16 : v; }

template <typename T>
__global__ void dequantize_kernel(const int8_t* __restrict__ q, const float* __restrict__ params, T* __restrict__ out,
                                  long long total, int group_size, int bits, int asym) {
  const int half = 1 << (bits - 1);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long g = i / group_size;
    const float s = params[g * (asym ? 2 : 1)], off = asym ? params[g * 2 + 1] : 0.f;
    int v;
    if (bits == 8) v = q[i];
    else {
      const int byte = q[i >> 1];
      v = sext4((i & 1) ? (byte >> 4) & 0xF : byte & 0xF);
    }
    out[i] = from_f32<T>(deq(v, s, off, asym, half));
  }
}

// out group g = requantised sum over `n_in` tensors' group g (all tensors share the group layout);
// input tensor t is at q_in + t * in_stride_bytes, params_in + t * groups * P.
__global__ void __launch_bounds__(256)
dequant_reduce_kernel(const int8_t* __restrict__ q_in, const float* __restrict__ p_in, int8_t* __restrict__ q_out,
                      float* __restrict__ p_out, int n_in, long long in_stride_bytes, int groups, int group_size,
                      int bits, int asym) {
  extern __shared__ float vals[];
  __shared__ float red[33];
  const int g = blockIdx.x, P = asym ? 2 : 1, half = 1 << (bits - 1), qmax = half - 1;
  float lo = INFINITY, hi = -INFINITY;
  for (int i = threadIdx.x; i < group_size; i += 256) {
    float acc = 0.f;
    for (int t = 0; t < n_in; ++t) {
      const int8_t* qt = q_in + t * in_stride_bytes;
      const float s = p_in[((long long)t * groups + g) * P], off = asym ? p_in[((long long)t * groups + g) * P + 1] : 0.f;
      int v;
      if (bits == 8) v = qt[(long long)g * group_size + i];
      else {
        const int byte = qt[((long long)g * group_size + i) >> 1];
        v = sext4((i & 1) ? (byte >> 4) & 0xF : byte & 0xF);
      }
      acc += deq(v, s, off, asym, half);
    }
    vals[i] = acc;
    lo = fminf(lo, acc);
    hi = fmaxf(hi, acc);
  }
  hi = block_max(hi, red);
  lo = -block_max(-lo, red);
  float s = asym ? (hi - lo) / (float)((1 << bits) - 1) : fmaxf(fabsf(hi), fabsf(lo)) / (float)qmax;
  const float off = asym ? lo : 0.f;
  if (s == 0.f) s = 1.f;
  if (threadIdx.x == 0) {
    p_out[(long long)g * P] = s;
    if (asym) p_out[(long long)g * P + 1] = off;
  }
  __syncthreads();
  const float inv = 1.f / s;
  if (bits == 8) {
    for (int i = threadIdx.x; i < group_size; i += 256)
      q_out[(long long)g * group_size + i] =
          (int8_t)fminf(fmaxf(rintf((vals[i] - off) * inv) - (asym ? half : 0), -half), qmax);
  } else {
    for (int i = threadIdx.x; i < group_size / 2; i += 256) {
      const int a = (int)fminf(fmaxf(rintf((vals[2 * i] - off) * inv) - (asym ? half : 0), -half), qmax) & 0xF;
      const int b = (int)fminf(fmaxf(rintf((vals[2 * i + 1] - off) * inv) - (asym ? half : 0), -half), qmax) & 0xF;
      q_out[(long long)g * (group_size / 2) + i] = (int8_t)(a | (b << 4));
    }
  }
}

// ---- optimizer-state codes ---------------------------------------------------------------
ATB_DEVICE uint32_t philox_hash(uint64_t seed, uint64_t idx) {   // counter-based, reproducible per element
  uint64_t z = seed + idx * 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return (uint32_t)((z ^ (z >> 31)) >> 32);
}

// absmax-linear: code = rint(x / absmax(group) * qmax) stored as int8 / int16; absmax per group
template <typename CODE>
__global__ void __launch_bounds__(256) pack_linear_kernel(const float* __restrict__ x, CODE* __restrict__ code,
                                                          float* __restrict__ absmax, long long n, int group_size,
                                                          int qmax) {
  __shared__ float red[33];
  const long long g0 = (long long)blockIdx.x * group_size;
  float am = 0.f;
  for (int i = threadIdx.x; i < group_size && g0 + i < n; i += 256) am = fmaxf(am, fabsf(x[g0 + i]));
  am = block_max(am, red);
  if (threadIdx.x == 0) absmax[blockIdx.x] = am;
  const float inv = am > 0.f ? (float)qmax / am : 0.f;
  for (int i = threadIdx.x; i < group_size && g0 + i < n; i += 256) code[g0 + i] = (CODE)rintf(x[g0 + i] * inv);
}
template <typename CODE>
__global__ void unpack_linear_kernel(const CODE* __restrict__ code, const float* __restrict__ absmax,
                                     float* __restrict__ out, long long n, int group_size, int qmax) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    out[i] = (float)code[i] * absmax[i / group_size] / (float)qmax;
}

// nonlinear: x / absmax(group) in [-1, 1] is mapped to the nearest entry of a sorted table `qmap`
// (2^bits entries); with stochastic rounding the two neighbours are chosen with probability
// proportional to proximity. 4-bit codes are packed two per byte.
__global__ void __launch_bounds__(256)
pack_nonlinear_kernel(const float* __restrict__ x, uint8_t* __restrict__ code, float* __restrict__ absmax,
                      const float* __restrict__ qmap, long long n, int group_size, int bits, int stochastic,
                      unsigned long long seed) {
  __shared__ float red[33];
  __shared__ float smap[256];
  const int nq = 1 << bits;
  for (int i = threadIdx.x; i < nq; i += 256) smap[i] = qmap[i];
  const long long g0 = (long long)blockIdx.x * group_size;
  float am = 0.f;
  for (int i = threadIdx.x; i < group_size && g0 + i < n; i += 256) am = fmaxf(am, fabsf(x[g0 + i]));
  am = block_max(am, red);
  if (threadIdx.x == 0) absmax[blockIdx.x] = am;
  const float inv = am > 0.f ? 1.f / am : 0.f;
  auto encode = [&](long long idx) -> int {
    if (idx >= n) return 0;
    const float v = x[idx] * inv;
    int lo = 0, hi = nq - 1;           // binary search: largest entry <= v
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (smap[mid] <= v) lo = mid; else hi = mid - 1;
    }
    if (lo == nq - 1) return lo;
    const float a = smap[lo], b = smap[lo + 1];
    if (stochastic) {
      const float u = (philox_hash(seed, (uint64_t)idx) >> 8) * (1.f / 16777216.f);
      return (v - a) > u * (b - a) ? lo + 1 : lo;
    }
    return (v - a) > (b - v) ? lo + 1 : lo;
  };
  if (bits == 8) {
    for (int i = threadIdx.x; i < group_size && g0 + i < n; i += 256) code[g0 + i] = (uint8_t)encode(g0 + i);
  } else {
    for (int i = threadIdx.x; i < group_size / 2 && g0 + 2 * i < n; i += 256)
      code[(g0 >> 1) + i] = (uint8_t)(encode(g0 + 2 * i) | (encode(g0 + 2 * i + 1) << 4));
  }
}
__global__ void unpack_nonlinear_kernel(const uint8_t* __restrict__ code, const float* __restrict__ absmax,
                                        const float* __restrict__ qmap, float* __restrict__ out, long long n,
                                        int group_size, int bits) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    int c;
    if (bits == 8) c = code[i];
    else c = (i & 1) ? code[i >> 1] >> 4 : code[i >> 1] & 0xF;
    out[i] = qmap[c] * absmax[i / group_size];
  }
}

inline int cap_grid(long long work, int threads) {
  long long g = (work + threads - 1) / threads;
  const long long cap = 148LL * 16;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}
}  // namespace

// dtype: 0 bf16, 1 fp16, 2 fp32. `group_map` (optional int32[groups]) redirects group g to output slot group_map[g].
extern "C" int atb_quantize(const void* x, void* q, float* params, int groups, int group_size, int bits, int asym,
                            const int* group_map, int dtype, void* stream) {
  if (groups <= 0) return 0;
  if ((bits != 4 && bits != 8) || (bits == 4 && (group_size & 1))) return -1;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == 0) quantize_kernel<__nv_bfloat16><<<groups, 256, 0, st>>>((const __nv_bfloat16*)x, (int8_t*)q, params, group_size, bits, asym, group_map, groups);
  else if (dtype == 1) quantize_kernel<__half><<<groups, 256, 0, st>>>((const __half*)x, (int8_t*)q, params, group_size, bits, asym, group_map, groups);
  else quantize_kernel<float><<<groups, 256, 0, st>>>((const float*)x, (int8_t*)q, params, group_size, bits, asym, group_map, groups);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
extern "C" int atb_dequantize(const void* q, const float* params, void* out, long long total, int group_size, int bits,
                              int asym, int dtype, void* stream) {
  if (total <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  const int g = cap_grid(total, 256);
  if (dtype == 0) dequantize_kernel<__nv_bfloat16><<<g, 256, 0, st>>>((const int8_t*)q, params, (__nv_bfloat16*)out, total, group_size, bits, asym);
  else if (dtype == 1) dequantize_kernel<__half><<<g, 256, 0, st>>>((const int8_t*)q, params, (__half*)out, total, group_size, bits, asym);
  else dequantize_kernel<float><<<g, 256, 0, st>>>((const int8_t*)q, params, (float*)out, total, group_size, bits, asym);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
extern "C" int atb_dequant_reduce(const void* q_in, const float* p_in, void* q_out, float* p_out, int n_in,
                                  long long in_stride_bytes, int groups, int group_size, int bits, int asym,
                                  void* stream) {
  if (groups <= 0) return 0;
  if (group_size * 4 > 160 * 1024) return -1;
  static bool attr = false;
  if (!attr) {
    cudaFuncSetAttribute(dequant_reduce_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
    attr = true;
  }
  dequant_reduce_kernel<<<groups, 256, group_size * 4, (cudaStream_t)stream>>>(
      (const int8_t*)q_in, p_in, (int8_t*)q_out, p_out, n_in, in_stride_bytes, groups, group_size, bits, asym);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
extern "C" int atb_pack_linear(const float* x, void* code, float* absmax, long long n, int group_size, int bits,
                               void* stream) {
  if (n <= 0) return 0;
  const int groups = (int)((n + group_size - 1) / group_size);
  if (bits == 8) pack_linear_kernel<int8_t><<<groups, 256, 0, (cudaStream_t)stream>>>(x, (int8_t*)code, absmax, n, group_size, 127);
  else if (bits == 16) pack_linear_kernel<int16_t><<<groups, 256, 0, (cudaStream_t)stream>>>(x, (int16_t*)code, absmax, n, group_size, 32767);
  else return -1;
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
extern "C" int atb_unpack_linear(const void* code, const float* absmax, float* out, long long n, int group_size,
                                 int bits, void* stream) {
  if (n <= 0) return 0;
  const int g = cap_grid(n, 256);
  if (bits == 8) unpack_linear_kernel<int8_t><<<g, 256, 0, (cudaStream_t)stream>>>((const int8_t*)code, absmax, out, n, group_size, 127);
  else if (bits == 16) unpack_linear_kernel<int16_t><<<g, 256, 0, (cudaStream_t)stream>>>((const int16_t*)code, absmax, out, n, group_size, 32767);
  else return -1;
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
extern "C" int atb_pack_nonlinear(const float* x, void* code, float* absmax, const float* qmap, long long n,
                                  int group_size, int bits, int stochastic, unsigned long long seed, void* stream) {
  if (n <= 0) return 0;
  if ((bits != 4 && bits != 8) || (bits == 4 && (group_size & 1))) return -1;
  const int groups = (int)((n + group_size - 1) / group_size);
  pack_nonlinear_kernel<<<groups, 256, 0, (cudaStream_t)stream>>>(x, (uint8_t*)code, absmax, qmap, n, group_size, bits, stochastic, seed);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
extern "C" int atb_unpack_nonlinear(const void* code, const float* absmax, const float* qmap, float* out, long long n,
                                    int group_size, int bits, void* stream) {
  if (n <= 0) return 0;
  unpack_nonlinear_kernel<<<cap_grid(n, 256), 256, 0, (cudaStream_t)stream>>>((const uint8_t*)code, absmax, qmap, out, n, group_size, bits);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
