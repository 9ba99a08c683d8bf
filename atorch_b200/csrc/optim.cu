// Fused flat-buffer optimizer steps for sm_100a: AdamW and AGD over a sharded fp32 master
// buffer, reading bf16 or fp32 gradients and writing the bf16 (or fp32) working copy of the
// parameters in the same pass. One read of (grad, master, m, v), one write of (master, m, v,
// param): 16-byte vectors, grid-stride.
//
// The optional `inv_scale_ptr` / `found_inf` pair implements the unscale + overflow check of
// mixed-precision loss scaling inside the same kernel (skip is decided by the caller after the
// inf check kernel). `grad_scale` folds gradient averaging and clipping into the update.
//
// Counterparts in the reference: torch.optim.AdamW under FSDP (examples/llama2), the Python AGD
// step in atorch/optimizers/agd.py:73-155, BF16Optimizer in atorch/optimizers/bf16_optimizer.py.
#include "common.cuh"

namespace {
using namespace atb;

template <typename G>
ATB_DEVICE void ldg4(const G* p, float (&v)[4]);
template <>
ATB_DEVICE void ldg4<float>(const float* p, float (&v)[4]) {
  float4 a = *reinterpret_cast<const float4*>(p);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
}
template <>
ATB_DEVICE void ldg4<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[4]) {
  uint2 u = *reinterpret_cast<const uint2*>(p);
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y);
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}

struct AdamArgs {
  float lr, beta1, beta2, eps, weight_decay, bc1, bc2;  // bc = 1 - beta^t
  float grad_scale;                                       // multiplies every gradient first
  int adamw;                                              // 1 decoupled decay, 0 L2 into the gradient
};

template <typename G>
__global__ void adamw_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                             const G* __restrict__ grad, __nv_bfloat16* __restrict__ param_bf16, long long n,
                             AdamArgs a, const float* __restrict__ grad_scale_ptr) {
  const float gs = a.grad_scale * (grad_scale_ptr ? *grad_scale_ptr : 1.f);
  const long long n4 = n >> 2;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4;
       i += (long long)gridDim.x * blockDim.x) {
    float g[4];
    ldg4<G>(grad + i * 4, g);
    float4 p4 = reinterpret_cast<float4*>(master)[i];
    float4 m4 = reinterpret_cast<float4*>(m)[i];
    float4 v4 = reinterpret_cast<float4*>(v)[i];
    float p[4] = {p4.x, p4.y, p4.z, p4.w}, mm[4] = {m4.x, m4.y, m4.z, m4.w}, vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float gj = g[j] * gs;
      if (a.adamw) p[j] *= (1.f - a.lr * a.weight_decay);
      else gj += a.weight_decay * p[j];
      mm[j] = a.beta1 * mm[j] + (1.f - a.beta1) * gj;
      vv[j] = a.beta2 * vv[j] + (1.f - a.beta2) * gj * gj;
      const float denom = sqrtf(vv[j] / a.bc2) + a.eps;
      p[j] -= a.lr * (mm[j] / a.bc1) / denom;
    }
    reinterpret_cast<float4*>(master)[i] = make_float4(p[0], p[1], p[2], p[3]);
    reinterpret_cast<float4*>(m)[i] = make_float4(mm[0], mm[1], mm[2], mm[3]);
    reinterpret_cast<float4*>(v)[i] = make_float4(vv[0], vv[1], vv[2], vv[3]);
    if (param_bf16) {
      uint2 o;
      o.x = pack_bf16x2(p[0], p[1]);
      o.y = pack_bf16x2(p[2], p[3]);
      reinterpret_cast<uint2*>(param_bf16)[i] = o;
    }
  }
  // tail (n not a multiple of 4)
  if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {
    const long long i = (n4 << 2) + threadIdx.x;
    float gj = to_f32<G>(grad[i]) * gs, p = master[i], mm = m[i], vv = v[i];
    if (a.adamw) p *= (1.f - a.lr * a.weight_decay);
    else gj += a.weight_decay * p;
    mm = a.beta1 * mm + (1.f - a.beta1) * gj;
    vv = a.beta2 * vv + (1.f - a.beta2) * gj * gj;
    p -= a.lr * (mm / a.bc1) / (sqrtf(vv / a.bc2) + a.eps);
    master[i] = p; m[i] = mm; v[i] = vv;
    if (param_bf16) param_bf16[i] = __float2bfloat16_rn(p);
  }
}

// AGD (atorch/optimizers/agd.py): s = m_t/(1-b1^t) - m_{t-1}/(1-b1^{t-1}) (t=1: m_t/(1-b1));
// v = b2 v + (1-b2) s^2; den = max(sqrt(v), delta*sqrt(1-b2^t)); u = m/den (optional clamp);
// p -= lr*sqrt(1-b2^t)/(1-b1^t) * u, with decoupled or L2 weight decay.
struct AgdArgs {
  float lr, beta1, beta2, delta, weight_decay;
  float bc1, bc1_old, bc2;  // 1-b1^t, 1-b1^(t-1) (unused at t=1), 1-b2^t
  float grad_scale, clip;   // clip <= 0: no clamp
  int first_step, decouple, fixed_decay;
};

ATB_DEVICE void agd_update(float& p, float& mm, float& vv, float g, const AgdArgs& a, float step_size, float dfloor) {
  if (a.decouple) p *= a.fixed_decay ? (1.f - a.weight_decay) : (1.f - a.lr * a.weight_decay);
  else g += a.weight_decay * p;
  const float m_old = mm;
  mm = a.beta1 * mm + (1.f - a.beta1) * g;
  const float s = a.first_step ? mm / a.bc1 : (mm / a.bc1 - m_old / a.bc1_old);
  vv = a.beta2 * vv + (1.f - a.beta2) * s * s;
  const float den = fmaxf(sqrtf(vv), dfloor);
  float u = mm / den;
  if (a.clip > 0.f) u = fminf(fmaxf(u, -a.clip), a.clip);
  p -= step_size * u;
}

template <typename G>
__global__ void agd_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                           const G* __restrict__ grad, __nv_bfloat16* __restrict__ param_bf16, long long n, AgdArgs a,
                           const float* __restrict__ grad_scale_ptr) {
  const float gs = a.grad_scale * (grad_scale_ptr ? *grad_scale_ptr : 1.f);
  const float step_size = a.lr * sqrtf(a.bc2) / a.bc1;
  const float dfloor = a.delta * sqrtf(a.bc2);
  const long long n4 = n >> 2;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4;
       i += (long long)gridDim.x * blockDim.x) {
    float g[4];
    ldg4<G>(grad + i * 4, g);
    float4 p4 = reinterpret_cast<float4*>(master)[i];
    float4 m4 = reinterpret_cast<float4*>(m)[i];
    float4 v4 = reinterpret_cast<float4*>(v)[i];
    float p[4] = {p4.x, p4.y, p4.z, p4.w}, mm[4] = {m4.x, m4.y, m4.z, m4.w}, vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) agd_update(p[j], mm[j], vv[j], g[j] * gs, a, step_size, dfloor);
    reinterpret_cast<float4*>(master)[i] = make_float4(p[0], p[1], p[2], p[3]);
    reinterpret_cast<float4*>(m)[i] = make_float4(mm[0], mm[1], mm[2], mm[3]);
    reinterpret_cast<float4*>(v)[i] = make_float4(vv[0], vv[1], vv[2], vv[3]);
    if (param_bf16) {
      uint2 o;
      o.x = pack_bf16x2(p[0], p[1]);
      o.y = pack_bf16x2(p[2], p[3]);
      reinterpret_cast<uint2*>(param_bf16)[i] = o;
    }
  }
  if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {   // tail (n not a multiple of 4)
    const long long i = (n4 << 2) + threadIdx.x;
    float p = master[i], mm = m[i], vv = v[i];
    agd_update(p, mm, vv, to_f32<G>(grad[i]) * gs, a, step_size, dfloor);
    master[i] = p; m[i] = mm; v[i] = vv;
    if (param_bf16) param_bf16[i] = __float2bfloat16_rn(p);
  }
}

// Sum of squares of a flat buffer into out[0] (fp32 atomics on one word per CTA; callers that
// need bit-reproducibility use the two-pass variant through partial[gridDim.x]).
template <typename G>
__global__ void sumsq_kernel(const G* __restrict__ x, long long n, float* __restrict__ partial) {
  __shared__ float red[33];
  float s = 0.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float v = to_f32<G>(x[i]);
    s += v * v;
  }
  s = block_sum(s, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}

// Nesterov / momentum SGD outer step of local SGD on a flat shard:
//   g = pseudo-gradient (already reduced); buf = mu*buf + g; p_sync -= lr*(g + mu*buf) (nesterov)
//   or p_sync -= lr*buf; then param <- p_sync.
__global__ void outer_sgd_kernel(float* __restrict__ synced, float* __restrict__ buf, const float* __restrict__ pg,
                                 float* __restrict__ param_f32, __nv_bfloat16* __restrict__ param_bf16, long long n,
                                 float lr, float mu, int nesterov, int first, float scale) {
  const long long n4 = n >> 2;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4;
       i += (long long)gridDim.x * blockDim.x) {
    const float4 g4 = reinterpret_cast<const float4*>(pg)[i];
    const float4 s4 = reinterpret_cast<const float4*>(synced)[i];
    float4 b4 = first ? make_float4(0.f, 0.f, 0.f, 0.f) : reinterpret_cast<const float4*>(buf)[i];
    float g[4] = {g4.x * scale, g4.y * scale, g4.z * scale, g4.w * scale};
    float b[4] = {b4.x, b4.y, b4.z, b4.w}, p[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      b[j] = first ? g[j] : mu * b[j] + g[j];
      p[j] -= lr * (nesterov ? (g[j] + mu * b[j]) : b[j]);
    }
    reinterpret_cast<float4*>(buf)[i] = make_float4(b[0], b[1], b[2], b[3]);
    reinterpret_cast<float4*>(synced)[i] = make_float4(p[0], p[1], p[2], p[3]);
    if (param_f32) reinterpret_cast<float4*>(param_f32)[i] = make_float4(p[0], p[1], p[2], p[3]);
    if (param_bf16) {
      uint2 o;
      o.x = pack_bf16x2(p[0], p[1]);
      o.y = pack_bf16x2(p[2], p[3]);
      reinterpret_cast<uint2*>(param_bf16)[i] = o;
    }
  }
  if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {
    const long long i = (n4 << 2) + threadIdx.x;
    const float g = pg[i] * scale;
    const float b = first ? g : mu * buf[i] + g;
    buf[i] = b;
    const float p = synced[i] - lr * (nesterov ? (g + mu * b) : b);
    synced[i] = p;
    if (param_f32) param_f32[i] = p;
    if (param_bf16) param_bf16[i] = __float2bfloat16_rn(p);
  }
}

inline int grid_for(long long work, int threads) {
  long long g = (work + threads - 1) / threads;
  long long cap = 148LL * 8;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}
}  // namespace

// grad_dtype: 0 bf16, 2 fp32. Buffers must be 16-byte aligned.
extern "C" int atb_adamw(float* master, float* m, float* v, const void* grad, void* param_bf16, long long n, float lr,
                         float beta1, float beta2, float eps, float weight_decay, int step, float grad_scale,
                         const float* grad_scale_ptr, int adamw_mode, int grad_dtype, int max_blocks, void* stream) {
  if (n <= 0) return 0;
  AdamArgs a{lr, beta1, beta2, eps, weight_decay, 1.f - powf(beta1, (float)step), 1.f - powf(beta2, (float)step),
             grad_scale, adamw_mode};
  int grid = grid_for((n + 3) / 4, 256);
  if (max_blocks > 0 && grid > max_blocks) grid = max_blocks;   // leave room for kernels sharing the SMs
  cudaStream_t st = (cudaStream_t)stream;
  if (grad_dtype == 0)
    adamw_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(master, m, v, (const __nv_bfloat16*)grad,
                                                     (__nv_bfloat16*)param_bf16, n, a, grad_scale_ptr);
  else
    adamw_kernel<float><<<grid, 256, 0, st>>>(master, m, v, (const float*)grad, (__nv_bfloat16*)param_bf16, n, a,
                                             grad_scale_ptr);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

extern "C" int atb_agd(float* master, float* m, float* v, const void* grad, void* param_bf16, long long n, float lr,
                       float beta1, float beta2, float delta, float weight_decay, int step, float grad_scale,
                       const float* grad_scale_ptr, float clip, int decouple, int fixed_decay, int grad_dtype,
                       void* stream) {
  if (n <= 0) return 0;
  // 16-byte vectors on the fp32 buffers, 8-byte on bf16 ones
  if ((((uintptr_t)master | (uintptr_t)m | (uintptr_t)v) & 15) || ((uintptr_t)param_bf16 & 7) ||
      ((uintptr_t)grad & (grad_dtype == 0 ? 7 : 15)))
    return -3;
  AgdArgs a{lr, beta1, beta2, delta, weight_decay, 1.f - powf(beta1, (float)step),
            step > 1 ? 1.f - powf(beta1, (float)(step - 1)) : 1.f, 1.f - powf(beta2, (float)step), grad_scale, clip,
            step == 1, decouple, fixed_decay};
  const int grid = grid_for((n + 3) / 4, 256);
  cudaStream_t st = (cudaStream_t)stream;
  if (grad_dtype == 0)
    agd_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(master, m, v, (const __nv_bfloat16*)grad,
                                                   (__nv_bfloat16*)param_bf16, n, a, grad_scale_ptr);
  else
    agd_kernel<float><<<grid, 256, 0, st>>>(master, m, v, (const float*)grad, (__nv_bfloat16*)param_bf16, n, a,
                                           grad_scale_ptr);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// partial must hold atb_sumsq_parts() floats; the caller sums them (fixed order).
extern "C" int atb_sumsq_parts() { return 148 * 4; }
extern "C" int atb_sumsq(const void* x, long long n, float* partial, int dtype, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  const int grid = atb_sumsq_parts();
  if (dtype == 0) sumsq_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, n, partial);
  else sumsq_kernel<float><<<grid, 256, 0, st>>>((const float*)x, n, partial);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

extern "C" int atb_outer_sgd(float* synced, float* buf, const float* pseudo_grad, float* param_f32, void* param_bf16,
                             long long n, float lr, float momentum, int nesterov, int first_step, float scale,
                             void* stream) {
  if (n <= 0) return 0;
  if ((((uintptr_t)synced | (uintptr_t)buf | (uintptr_t)pseudo_grad | (uintptr_t)param_f32) & 15) ||
      ((uintptr_t)param_bf16 & 7))
    return -3;
  outer_sgd_kernel<<<grid_for((n + 3) / 4, 256), 256, 0, (cudaStream_t)stream>>>(
      synced, buf, pseudo_grad, param_f32, (__nv_bfloat16*)param_bf16, n, lr, momentum, nesterov, first_step, scale);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
