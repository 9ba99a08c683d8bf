// Softmax cross-entropy forward / backward over [rows, vocab] logits for sm_100a, with
// ignore_index, label smoothing, z-loss (lse_square_scale * lse^2) and a vocabulary-split mode
// for tensor-parallel heads (each rank passes its vocabulary slice and offset; the per-rank
// lse values are combined by the caller and fed to the backward).
//
// One CTA per row; the row is streamed once with 16-byte loads through an online
// (max, sum-exp) reduction. The backward rewrites the logits in place if asked.
//
// Counterpart in the reference: atorch/kernels/triton_jit/cross_entropy.py:33-254 and
// atorch/modules/distributed_modules/cross_entropy.py:9-127.
#include "common.cuh"

namespace {
using namespace atb;
constexpr int CE_NT = 512;

template <typename T>
ATB_DEVICE void ld8(const T* p, float (&v)[8]);
template <>
ATB_DEVICE void ld8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
}
template <>
ATB_DEVICE void ld8<float>(const float* p, float (&v)[8]) {
  float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <typename T>
ATB_DEVICE void st8(T* p, const float (&v)[8]);
template <>
ATB_DEVICE void st8<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 u;
  u.x = pack_bf16x2(v[0], v[1]); u.y = pack_bf16x2(v[2], v[3]);
  u.z = pack_bf16x2(v[4], v[5]); u.w = pack_bf16x2(v[6], v[7]);
  *reinterpret_cast<uint4*>(p) = u;
}
template <>
ATB_DEVICE void st8<float>(float* p, const float (&v)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}

// Per row outputs: lse (local to this vocabulary slice), label_logit (0 if the label is not in
// the slice), sum_logits (for label smoothing), and, when `loss` != nullptr (single-slice use),
// the finished loss value.
template <typename T>
__global__ void __launch_bounds__(CE_NT) ce_fwd_kernel(const T* __restrict__ logits, const long long* __restrict__ labels,
                                                       float* __restrict__ loss, float* __restrict__ lse_out,
                                                       float* __restrict__ label_logit_out,
                                                       float* __restrict__ sum_logits_out, int V, long long stride,
                                                       int vocab_start, long long v_total, long long ignore_index,
                                                       float smoothing, float z_scale) {
  __shared__ float red[33];
  const long long row = blockIdx.x;
  const T* x = logits + row * stride;
  float m = -INFINITY, s = 0.f, tot = 0.f;
  const int nvec = V >> 3;
  // the label and its logit are fetched now, so that the two dependent loads are not a serial tail of the row
  long long lab = ignore_index;
  float ll = 0.f;
  if (threadIdx.x == 0) {
    lab = labels[row];
    const long long local = lab - vocab_start;
    if (lab != ignore_index && local >= 0 && local < V) ll = to_f32<T>(x[local]);
  }
  constexpr float L2E = 1.4426950408889634f;
  constexpr int U = 2;   // 16-byte loads in flight per thread; one rescale of the running sum per 16 elements
  for (int c0 = threadIdx.x; c0 < nvec; c0 += U * CE_NT) {
    float v[U][8];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int c = c0 + u * CE_NT;
      if (c < nvec) {
        ld8<T>(x + c * 8, v[u]);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[u][j] = -INFINITY;
      }
    }
    float lm = v[0][0];
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int j = 0; j < 8; ++j) lm = fmaxf(lm, v[u][j]);
    const float nm = fmaxf(m, lm);
    const float nms = (nm == -INFINITY) ? 0.f : -nm * L2E;
    float acc[2] = {0.f, 0.f};
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        acc[j & 1] += fast_exp2(fmaf(v[u][j], L2E, nms));          // exp(v - nm); -inf padding gives 0
        if (smoothing > 0.f && v[u][j] != -INFINITY) tot += v[u][j];
      }
    s = s * fast_exp2(fmaf(m, L2E, nms)) + (acc[0] + acc[1]);      // m = -inf: factor 0
    m = nm;
  }
  for (int c = (nvec << 3) + threadIdx.x; c < V; c += CE_NT) {  // ragged tail
    const float v = to_f32<T>(x[c]);
    const float nm = fmaxf(m, v);
    s = s * __expf(m - nm) + __expf(v - nm);
    m = nm;
    tot += v;
  }
  const float gm = block_max(m, red);
  s = (m == -INFINITY) ? 0.f : s * __expf(m - gm);
  s = block_sum(s, red);
  tot = block_sum(tot, red);
  if (threadIdx.x == 0) {
    const float lse = gm + logf(s);
    lse_out[row] = lse;
    if (label_logit_out) label_logit_out[row] = ll;
    if (sum_logits_out) sum_logits_out[row] = tot;
    if (loss) {
      float l = 0.f;
      if (lab != ignore_index) {
        l = (lse - ll) * (1.f - smoothing);
        if (smoothing > 0.f) l += smoothing * (lse - tot / (float)v_total);
        l += z_scale * lse * lse;
      }
      loss[row] = l;
    }
  }
}

// dlogits[j] = g * (p_j * (1 + 2 z lse) - (1 - eps) [j == label] - eps / V_total),  p_j = exp(x_j - lse)
// g = grad_scalar (if dloss == nullptr) else dloss[row]; rows with label == ignore_index get zeros.
template <typename T>
__global__ void __launch_bounds__(CE_NT) ce_bwd_kernel(const T* __restrict__ logits, const long long* __restrict__ labels,
                                                       const float* __restrict__ lse_in, const float* __restrict__ dloss,
                                                       float grad_scalar, T* __restrict__ dlogits, int V,
                                                       long long stride, int vocab_start, long long v_total,
                                                       long long ignore_index, float smoothing, float z_scale) {
  const long long row = blockIdx.x;
  const T* x = logits + row * stride;
  T* dx = dlogits + row * stride;
  const long long lab = labels[row];
  const bool ignored = lab == ignore_index;
  const float g = ignored ? 0.f : (dloss ? dloss[row] : grad_scalar);
  const float lse = lse_in[row];
  const float pscale = g * (1.f + 2.f * z_scale * lse);
  const float sm = g * smoothing / (float)v_total;
  const long long local = lab - vocab_start;
  const int nvec = V >> 3;
  for (int c = threadIdx.x; c < nvec; c += CE_NT) {
    float v[8];
    ld8<T>(x + c * 8, v);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float d = pscale * __expf(v[j] - lse) - sm;
      if ((long long)(c * 8 + j) == local) d -= g * (1.f - smoothing);
      v[j] = d;
    }
    st8<T>(dx + c * 8, v);
  }
  for (int c = (nvec << 3) + threadIdx.x; c < V; c += CE_NT) {
    float d = pscale * __expf(to_f32<T>(x[c]) - lse) - sm;
    if ((long long)c == local) d -= g * (1.f - smoothing);
    dx[c] = from_f32<T>(d);
  }
}
}  // namespace

// dtype: 0 = bf16, 2 = fp32. `stride` = row pitch in elements (multiple of 8).
extern "C" int atb_ce_fwd(const void* logits, const long long* labels, float* loss, float* lse, float* label_logit,
                          float* sum_logits, long long rows, int V, long long stride, int vocab_start,
                          long long v_total, long long ignore_index, float smoothing, float z_scale, int dtype,
                          void* stream) {
  if (rows <= 0) return 0;
  if (stride & 7) return -1;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == 0)
    ce_fwd_kernel<__nv_bfloat16><<<(unsigned)rows, CE_NT, 0, st>>>((const __nv_bfloat16*)logits, labels, loss, lse,
                                                                  label_logit, sum_logits, V, stride, vocab_start,
                                                                  v_total, ignore_index, smoothing, z_scale);
  else if (dtype == 2)
    ce_fwd_kernel<float><<<(unsigned)rows, CE_NT, 0, st>>>((const float*)logits, labels, loss, lse, label_logit,
                                                          sum_logits, V, stride, vocab_start, v_total, ignore_index,
                                                          smoothing, z_scale);
  else return -1;
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

extern "C" int atb_ce_bwd(const void* logits, const long long* labels, const float* lse, const float* dloss,
                          float grad_scalar, void* dlogits, long long rows, int V, long long stride, int vocab_start,
                          long long v_total, long long ignore_index, float smoothing, float z_scale, int dtype,
                          void* stream) {
  if (rows <= 0) return 0;
  if (stride & 7) return -1;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == 0)
    ce_bwd_kernel<__nv_bfloat16><<<(unsigned)rows, CE_NT, 0, st>>>((const __nv_bfloat16*)logits, labels, lse, dloss,
                                                                  grad_scalar, (__nv_bfloat16*)dlogits, V, stride,
                                                                  vocab_start, v_total, ignore_index, smoothing, z_scale);
  else if (dtype == 2)
    ce_bwd_kernel<float><<<(unsigned)rows, CE_NT, 0, st>>>((const float*)logits, labels, lse, dloss, grad_scalar,
                                                          (float*)dlogits, V, stride, vocab_start, v_total,
                                                          ignore_index, smoothing, z_scale);
  else return -1;
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
