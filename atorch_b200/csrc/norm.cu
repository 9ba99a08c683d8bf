// RMSNorm and LayerNorm, forward and backward, for sm_100a.
//
// Memory-bound row kernels: each CTA walks rows with a grid stride, a row lives in registers
// between the statistics pass and the output pass (one read of x, one write of y), all global
// accesses are 16-byte vectors. The weight/bias gradients are reduced deterministically in two
// passes: every CTA accumulates its rows into a private fp32 partial row of a scratch matrix
// [gridDim.x, N], then a column kernel sums the partial rows in a fixed order. No atomics, no
// spin locks, results are bit-reproducible.
//
// Counterparts in the reference: atorch/kernels/triton_jit/rmsnorm_kernel.py:8-214 (Triton,
// dw via a spin lock) and atorch/kernels/triton_jit/atorch_layer_norm.py:20-260.
#include "common.cuh"
#include <type_traits>

namespace {
using namespace atb;

constexpr int NT = 256;  // threads per CTA

template <typename T>
struct Vec8 {
  uint4 raw;
};

template <typename T>
ATB_DEVICE void load8(const T* p, float (&v)[8]);
template <>
ATB_DEVICE void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
}
template <>
ATB_DEVICE void load8<__half>(const __half* p, float (&v)[8]) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __half22float2(h[i]);
    v[2 * i] = f.x; v[2 * i + 1] = f.y;
  }
}
template <>
ATB_DEVICE void load8<float>(const float* p, float (&v)[8]) {
  float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <typename T>
ATB_DEVICE void store8(T* p, const float (&v)[8]);
template <>
ATB_DEVICE void store8<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 u;
  u.x = pack_bf16x2(v[0], v[1]); u.y = pack_bf16x2(v[2], v[3]);
  u.z = pack_bf16x2(v[4], v[5]); u.w = pack_bf16x2(v[6], v[7]);
  *reinterpret_cast<uint4*>(p) = u;
}
template <>
ATB_DEVICE void store8<__half>(__half* p, const float (&v)[8]) {
  uint4 u;
  __half2* h = reinterpret_cast<__half2*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = u;
}
template <>
ATB_DEVICE void store8<float>(float* p, const float (&v)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}

// A row piece as loaded (8 elements, undecoded): what the software pipeline keeps in registers for the
// row after the current one, so that its loads are in flight during the reductions of this one.
template <typename T>
struct Raw8 {
  uint4 v[sizeof(T) / 2];
};
template <typename T>
ATB_DEVICE Raw8<T> ldraw(const T* p) {
  Raw8<T> r;
#pragma unroll
  for (int k = 0; k < (int)(sizeof(T) / 2); ++k) r.v[k] = reinterpret_cast<const uint4*>(p)[k];
  return r;
}
template <typename T>
ATB_DEVICE void decode8(const Raw8<T>& r, float (&v)[8]) {
  if constexpr (std::is_same<T, __nv_bfloat16>::value) {
    float2 a = unpack_bf16x2(r.v[0].x), b = unpack_bf16x2(r.v[0].y), c = unpack_bf16x2(r.v[0].z),
           d = unpack_bf16x2(r.v[0].w);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
  } else if constexpr (std::is_same<T, __half>::value) {
    const __half2* h = reinterpret_cast<const __half2*>(&r.v[0]);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __half22float2(h[i]);
      v[2 * i] = f.x; v[2 * i + 1] = f.y;
    }
  } else {
    v[0] = __uint_as_float(r.v[0].x); v[1] = __uint_as_float(r.v[0].y); v[2] = __uint_as_float(r.v[0].z);
    v[3] = __uint_as_float(r.v[0].w); v[4] = __uint_as_float(r.v[1].x); v[5] = __uint_as_float(r.v[1].y);
    v[6] = __uint_as_float(r.v[1].z); v[7] = __uint_as_float(r.v[1].w);
  }
}
// value after a round trip through the storage type (what a re-read of a stored tensor would give)
template <typename T>
ATB_DEVICE float round_through(float x) {
  if constexpr (std::is_same<T, __nv_bfloat16>::value) return __bfloat162float(__float2bfloat16_rn(x));
  else if constexpr (std::is_same<T, __half>::value) return __half2float(__float2half_rn(x));
  else return x;
}

// ------------------------------------------------------------------------------------------
// forward:  y = (x [+ residual]) * rstd * w           (LN: (x - mean) * rstd * w + b)
// If `residual` is given, the sum x + residual is also written to `sum_out` (pre-norm stream).
// ------------------------------------------------------------------------------------------
template <typename T, int VPT, bool LN, bool RES>
__global__ void __launch_bounds__(NT, (VPT <= 2 && !LN) ? 4 : 1) norm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ residual,
                                                      const T* __restrict__ w, const T* __restrict__ b,
                                                      T* __restrict__ y, T* __restrict__ sum_out,
                                                      float* __restrict__ mean_out, float* __restrict__ rstd_out,
                                                      int M, int N, float eps) {
  __shared__ float red[33];
  const int nvec = N >> 3;
  float wv[VPT][8], bv[VPT][8];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = threadIdx.x + i * NT;
    if (c < nvec) {
      load8<T>(w + c * 8, wv[i]);
      if (LN && b != nullptr) load8<T>(b + c * 8, bv[i]);
      else {
#pragma unroll
        for (int j = 0; j < 8; ++j) bv[i][j] = 0.f;
      }
    }
  }
  Raw8<T> nx[VPT], nr[RES ? VPT : 1];
  auto fetch = [&](int row) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = threadIdx.x + i * NT;
      if (c < nvec) {
        nx[i] = ldraw<T>(x + (size_t)row * N + c * 8);
        if constexpr (RES) nr[i] = ldraw<T>(residual + (size_t)row * N + c * 8);
      }
    }
  };
  if ((int)blockIdx.x < M) fetch(blockIdx.x);
  for (int row = blockIdx.x; row < M; row += gridDim.x) {
    float xv[VPT][8];
    float s = 0.f, ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = threadIdx.x + i * NT;
      if (c < nvec) {
        decode8<T>(nx[i], xv[i]);
        if constexpr (RES) {
          float rv[8];
          decode8<T>(nr[i], rv);
          // round through the storage type so the normalised value matches a re-read of sum_out
#pragma unroll
          for (int j = 0; j < 8; ++j) xv[i][j] = round_through<T>(xv[i][j] + rv[j]);
          store8<T>(sum_out + (size_t)row * N + c * 8, xv[i]);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          s += xv[i][j];
          ss += xv[i][j] * xv[i][j];
        }
      }
    }
    // the next row's loads are issued before this row's reductions
    if (row + (int)gridDim.x < M) fetch(row + gridDim.x);
    float mean = 0.f, rstd;
    if (LN) {
      mean = block_sum(s, red) / N;
      float var = 0.f;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int c = threadIdx.x + i * NT;
        if (c < nvec) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float d = xv[i][j] - mean;
            var += d * d;
          }
        }
      }
      var = block_sum(var, red) / N;
      rstd = rsqrtf(var + eps);
    } else {
      ss = block_sum(ss, red);
      rstd = rsqrtf(ss / N + eps);
    }
    if (threadIdx.x == 0) {
      rstd_out[row] = rstd;
      if (LN) mean_out[row] = mean;
    }
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = threadIdx.x + i * NT;
      if (c < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = (xv[i][j] - mean) * rstd * wv[i][j] + bv[i][j];
        store8<T>(y + (size_t)row * N + c * 8, o);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------
// backward: dx = (w*dy - xhat * mean(xhat*w*dy) [- mean(w*dy) for LN]) * rstd  [+ dres]
//           partial_dw[cta] = sum_rows dy * xhat ; partial_db[cta] = sum_rows dy
// ------------------------------------------------------------------------------------------
template <typename T, int VPT, bool LN>
__global__ void __launch_bounds__(NT) norm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                                      const T* __restrict__ w, const float* __restrict__ mean_in,
                                                      const float* __restrict__ rstd_in, const T* __restrict__ dres,
                                                      T* __restrict__ dx, float* __restrict__ partial_dw,
                                                      float* __restrict__ partial_db, int M, int N) {
  __shared__ float red[33];
  const int nvec = N >> 3;
  float wv[VPT][8], dwacc[VPT][8], dbacc[VPT][8];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = threadIdx.x + i * NT;
    if (c < nvec) load8<T>(w + c * 8, wv[i]);
#pragma unroll
    for (int j = 0; j < 8; ++j) { dwacc[i][j] = 0.f; dbacc[i][j] = 0.f; }
  }
  // contiguous row chunk per CTA keeps the partial sums' order independent of the grid stride
  const int rows_per = (M + gridDim.x - 1) / gridDim.x;
  const int r0 = blockIdx.x * rows_per, r1 = min(M, r0 + rows_per);
  Raw8<T> nx[VPT], ndy[VPT];
  auto fetch = [&](int row) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = threadIdx.x + i * NT;
      if (c < nvec) {
        nx[i] = ldraw<T>(x + (size_t)row * N + c * 8);
        ndy[i] = ldraw<T>(dy + (size_t)row * N + c * 8);
      }
    }
  };
  if (r0 < r1) fetch(r0);
  for (int row = r0; row < r1; ++row) {
    const float rstd = rstd_in[row];
    const float mean = LN ? mean_in[row] : 0.f;
    float xh[VPT][8], g[VPT][8];
    float c1 = 0.f, c2 = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = threadIdx.x + i * NT;
      if (c < nvec) {
        float xv[8], dyv[8];
        decode8<T>(nx[i], xv);
        decode8<T>(ndy[i], dyv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] = (xv[j] - mean) * rstd;
          g[i][j] = dyv[j] * wv[i][j];
          c1 += xh[i][j] * g[i][j];
          c2 += g[i][j];
          dwacc[i][j] += dyv[j] * xh[i][j];
          dbacc[i][j] += dyv[j];
        }
      }
    }
    if (row + 1 < r1) fetch(row + 1);   // in flight during the reductions and the store of this row
    c1 = block_sum(c1, red) / N;
    if (LN) c2 = block_sum(c2, red) / N; else c2 = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = threadIdx.x + i * NT;
      if (c < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = (g[i][j] - xh[i][j] * c1 - c2) * rstd;
        if (dres != nullptr) {
          float rv[8];
          load8<T>(dres + (size_t)row * N + c * 8, rv);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += rv[j];
        }
        store8<T>(dx + (size_t)row * N + c * 8, o);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = threadIdx.x + i * NT;
    if (c < nvec) {
      store8<float>(partial_dw + (size_t)blockIdx.x * N + c * 8, dwacc[i]);
      if (LN && partial_db != nullptr) store8<float>(partial_db + (size_t)blockIdx.x * N + c * 8, dbacc[i]);
    }
  }
}

// out[c] (+)= sum_p partial[p][c]; fixed summation order. A CTA owns 32 columns; its 8 row groups (thread
// group g takes rows g, g+8, ...) each keep two running sums and are combined through shared memory in a
// fixed order, so the result does not depend on scheduling while 8 x more loads are in flight per column
// than with one thread per column.
constexpr int CS_COLS = 32, CS_GROUPS = 8;
template <typename TO>
__global__ void __launch_bounds__(CS_COLS * CS_GROUPS)
colsum_kernel(const float* __restrict__ partial, TO* __restrict__ out, int P, int N, int accumulate) {
  __shared__ float part[CS_GROUPS][CS_COLS];
  const int cl = threadIdx.x % CS_COLS, g = threadIdx.x / CS_COLS;
  const int c = blockIdx.x * CS_COLS + cl;
  float s0 = 0.f, s1 = 0.f;
  if (c < N) {
    int p = g;
    for (; p + CS_GROUPS < P; p += 2 * CS_GROUPS) {
      s0 += partial[(size_t)p * N + c];
      s1 += partial[(size_t)(p + CS_GROUPS) * N + c];
    }
    if (p < P) s0 += partial[(size_t)p * N + c];
  }
  part[g][cl] = s0 + s1;
  __syncthreads();
  if (g == 0 && c < N) {
    float s = ((part[0][cl] + part[1][cl]) + (part[2][cl] + part[3][cl])) +
              ((part[4][cl] + part[5][cl]) + (part[6][cl] + part[7][cl]));
    if (accumulate) s += to_f32<TO>(out[c]);
    out[c] = from_f32<TO>(s);
  }
}

template <typename T, bool LN>
int launch_fwd(const void* x, const void* res, const void* w, const void* b, void* y, void* sum_out, float* mean,
               float* rstd, int M, int N, float eps, cudaStream_t st) {
  const int nvec = N >> 3;
  const int vpt = (nvec + NT - 1) / NT;
  int grid = M < 148 * 8 ? M : 148 * 8;
#define L(V)                                                                                                       \
  do {                                                                                                             \
    if (res != nullptr)                                                                                            \
      norm_fwd_kernel<T, V, LN, true><<<grid, NT, 0, st>>>((const T*)x, (const T*)res, (const T*)w, (const T*)b,   \
                                                           (T*)y, (T*)sum_out, mean, rstd, M, N, eps);            \
    else                                                                                                           \
      norm_fwd_kernel<T, V, LN, false><<<grid, NT, 0, st>>>((const T*)x, (const T*)res, (const T*)w, (const T*)b,  \
                                                            (T*)y, (T*)sum_out, mean, rstd, M, N, eps);           \
  } while (0)
  if (vpt <= 1) L(1);
  else if (vpt <= 2) L(2);
  else if (vpt <= 4) L(4);
  else if (vpt <= 8) L(8);
  else return -1;
#undef L
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

template <typename T, bool LN>
int launch_bwd(const void* dy, const void* x, const void* w, const float* mean, const float* rstd, const void* dres,
               void* dx, float* pdw, float* pdb, int parts, int M, int N, cudaStream_t st) {
  const int nvec = N >> 3;
  const int vpt = (nvec + NT - 1) / NT;
#define L(V)                                                                                                    \
  norm_bwd_kernel<T, V, LN><<<parts, NT, 0, st>>>((const T*)dy, (const T*)x, (const T*)w, mean, rstd,          \
                                                  (const T*)dres, (T*)dx, pdw, pdb, M, N)
  if (vpt <= 1) L(1);
  else if (vpt <= 2) L(2);
  else if (vpt <= 4) L(4);
  else return -1;
#undef L
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

}  // namespace

// dtype: 0 = bf16, 1 = fp16, 2 = fp32.  N % 8 == 0, N <= 16384 (fwd) / 8192 (bwd).
extern "C" int atb_norm_fwd(const void* x, const void* residual, const void* w, const void* b, void* y, void* sum_out,
                            float* mean, float* rstd, int M, int N, float eps, int layernorm, int dtype,
                            void* stream) {
  if (M <= 0) return 0;
  if (N & 7) return -1;
  cudaStream_t st = (cudaStream_t)stream;
#define D(T)                                                                                               \
  return layernorm ? launch_fwd<T, true>(x, residual, w, b, y, sum_out, mean, rstd, M, N, eps, st)        \
                   : launch_fwd<T, false>(x, residual, w, b, y, sum_out, mean, rstd, M, N, eps, st)
  if (dtype == 0) D(__nv_bfloat16);
  if (dtype == 1) D(__half);
  if (dtype == 2) D(float);
#undef D
  return -1;
}

// Number of partial rows the backward wants for a given M (scratch is [parts, N] fp32, twice for LN).
extern "C" int atb_norm_bwd_parts(int M) {
  int p = 148 * 2;
  return M < p ? M : p;
}

extern "C" int atb_norm_bwd(const void* dy, const void* x, const void* w, const float* mean, const float* rstd,
                            const void* dres, void* dx, float* partial_dw, float* partial_db, int parts, int M, int N,
                            int layernorm, int dtype, void* stream) {
  if (M <= 0) return 0;
  if (N & 7) return -1;
  cudaStream_t st = (cudaStream_t)stream;
#define D(T)                                                                                                     \
  return layernorm ? launch_bwd<T, true>(dy, x, w, mean, rstd, dres, dx, partial_dw, partial_db, parts, M, N, st) \
                   : launch_bwd<T, false>(dy, x, w, mean, rstd, dres, dx, partial_dw, partial_db, parts, M, N, st)
  if (dtype == 0) D(__nv_bfloat16);
  if (dtype == 1) D(__half);
  if (dtype == 2) D(float);
#undef D
  return -1;
}

// out[N] (+)= column sums of partial[P, N].  out_dtype: 0 bf16, 1 fp16, 2 fp32.
extern "C" int atb_colsum(const float* partial, void* out, int P, int N, int out_dtype, int accumulate, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  const int grid = (N + CS_COLS - 1) / CS_COLS, threads = CS_COLS * CS_GROUPS;
  if (out_dtype == 0) colsum_kernel<__nv_bfloat16><<<grid, threads, 0, st>>>(partial, (__nv_bfloat16*)out, P, N, accumulate);
  else if (out_dtype == 1) colsum_kernel<__half><<<grid, threads, 0, st>>>(partial, (__half*)out, P, N, accumulate);
  else colsum_kernel<float><<<grid, threads, 0, st>>>(partial, (float*)out, P, N, accumulate);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// ------------------------------------------------------------------------------------------------
// Allocation-free RMSNorm backward (declared in no_alloc.h).
//
// Some callers of this library cannot allocate device memory around a kernel: code that runs inside
// a region where cudaMalloc is forbidden or deadlocks (a memory pool owned by another runtime, a
// pre-sized inference/training arena, a callback or a latency-critical path that must not touch the
// allocator, or a host framework that hands out only the input and output buffers). The regular
// backward needs a [parts, N] fp32 scratch matrix for the deterministic weight-gradient reduction,
// which the PyTorch wrapper allocates per call. This variant keeps that scratch in a file-scope
// device array instead, so the caller passes inputs and outputs only.
//
// The array is NA_MAX_PARTS * NA_MAX_N floats (148 * 8192 * 4 B = 4.6 MiB) and is held by every GPU
// that loads the library, until the process exits. Sizes beyond it (N > 8192) are rejected.
// ------------------------------------------------------------------------------------------------
#include <mutex>
#include <cstdio>
#include "no_alloc.h"   // the declarations below must match the header that callers compile against

namespace {
constexpr int NA_MAX_PARTS = 148;   // one partial row per SM
constexpr int NA_MAX_N = 8192;
constexpr int NA_MAX_DEVICES = 64;
thread_local char g_na_error[256] = "";
}  // namespace

static __device__ __align__(256) float g_na_scratch[NA_MAX_PARTS * NA_MAX_N];

namespace {
// In host code `g_na_scratch` is only a stand-in for the symbol, not a device address; the address
// that kernels may use is looked up once per device, with that device current.
float* na_scratch_address() {
  static std::mutex mu;
  static float* ptrs[NA_MAX_DEVICES] = {nullptr};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= NA_MAX_DEVICES) {
    snprintf(g_na_error, sizeof(g_na_error), "no current CUDA device (or device index >= %d)", NA_MAX_DEVICES);
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (ptrs[dev] == nullptr) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_na_scratch);
    if (e != cudaSuccess || p == nullptr) {
      snprintf(g_na_error, sizeof(g_na_error), "cudaGetSymbolAddress failed on device %d: %s", dev,
               cudaGetErrorString(e));
      return nullptr;
    }
    ptrs[dev] = static_cast<float*>(p);
  }
  return ptrs[dev];
}
}  // namespace

extern "C" const char* atb_noalloc_last_error() { return g_na_error; }

extern "C" int atb_noalloc_max_n() { return NA_MAX_N; }

extern "C" int atb_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, void* dx,
                                       void* dw, int M, int N, int dtype, void* stream) {
  g_na_error[0] = 0;
  if (M <= 0 || N <= 0) {
    snprintf(g_na_error, sizeof(g_na_error), "M and N must be positive (got M=%d N=%d)", M, N);
    return -10;
  }
  if (N > NA_MAX_N) {
    snprintf(g_na_error, sizeof(g_na_error), "N=%d exceeds the built-in scratch limit of %d columns", N, NA_MAX_N);
    return -11;
  }
  if (N & 7) {
    snprintf(g_na_error, sizeof(g_na_error), "N=%d must be a multiple of 8", N);
    return -12;
  }
  if (dtype < 0 || dtype > 2) {
    snprintf(g_na_error, sizeof(g_na_error), "dtype %d is not 0 (bf16), 1 (fp16) or 2 (fp32)", dtype);
    return -13;
  }
  float* scratch = na_scratch_address();
  if (scratch == nullptr) return -14;
  const int parts = M < NA_MAX_PARTS ? M : NA_MAX_PARTS;
  cudaStream_t st = (cudaStream_t)stream;
  int rc;
  // Every one of the `parts` partial rows is fully written by its CTA before the column sum reads
  // it, so nothing has to be cleared between calls even though the array keeps old contents.
  if (dtype == 0)
    rc = launch_bwd<__nv_bfloat16, false>(dy, x, w, nullptr, rstd, nullptr, dx, scratch, nullptr, parts, M, N, st);
  else if (dtype == 1)
    rc = launch_bwd<__half, false>(dy, x, w, nullptr, rstd, nullptr, dx, scratch, nullptr, parts, M, N, st);
  else
    rc = launch_bwd<float, false>(dy, x, w, nullptr, rstd, nullptr, dx, scratch, nullptr, parts, M, N, st);
  if (rc != 0) {
    snprintf(g_na_error, sizeof(g_na_error), "backward kernel launch failed (%d)", rc);
    return rc;
  }
  rc = atb_colsum(scratch, dw, parts, N, dtype, 0, stream);
  if (rc != 0) snprintf(g_na_error, sizeof(g_na_error), "column-sum kernel launch failed (%d)", rc);
  return rc;
}
