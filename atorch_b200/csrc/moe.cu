// Mixture-of-experts token exchange over NVLink peer memory for sm_100a: routing bookkeeping on the
// device, dispatch (scatter) straight into the destination ranks' expert buffers and combine (gather)
// straight out of them - the all-to-all of an expert-parallel layer without a collective call, a host
// sync, or a permuted intermediate copy.
//
// Buffers (symmetric: every rank maps every peer's copy):
//   expert buffer  X[e_local][src_rank][slot][H]   slot < capacity; only the first count[e_local][src] slots
//                  of a (e_local, src) group hold tokens, the rest is zero (atb_moe_zero_tail)
//   counts         C[e_local][src_rank]            written by the source rank together with its tokens
// Routing: entry i = (token t = i / k, choice j = i % k) goes to expert e = idx[i]; its slot is the number
// of earlier entries of this rank with the same expert (token order, deterministic); entries whose slot
// reaches the capacity are dropped (slot = -1), as with capacity-factor routing.
//
//   atb_moe_route    idx[T*k] -> slot[T*k], count[E] (clamped to the capacity)
//   atb_moe_scatter  rows of src[T, H] (optionally times w[i]) -> peer expert buffers; then the counts;
//                    the block that finishes last signals ARRIVE to every rank (pad protocol of comm.cu)
//   atb_moe_zero_tail zero the unused slots of every (e_local, src) group of the local buffer
//   atb_moe_gather   out[t] = sum_j w[i] * X_peer(e)[...][slot[i]]  (peer loads); optionally also
//                    dw[i] = <g[t], row> for the backward of the probability-weighted combine
//
// Replaces permute + all_to_all (+ second permute) and unpermute + all_to_all of the reference
// (atorch/modules/moe/token_dispatcher.py:297-470), whose split sizes go through the host.
#include "common.cuh"

namespace {
using namespace atb;

constexpr int MAX_RANKS = 8;

struct MoePeers {
  void* buf[MAX_RANKS];       // expert buffers (bf16)
  int* counts[MAX_RANKS];     // counts[e_local * world + src]
  uint32_t* pad[MAX_RANKS];   // signal pads
  unsigned int* counter;      // blocks finished (self-resetting)
  int rank, world;
  unsigned int seq;
};

__device__ unsigned long long g_moe_wait_ns = ATB_WAIT_LIMIT_NS;

ATB_DEVICE void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
ATB_DEVICE uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// One CTA per expert: positions of the entries routed to that expert, in entry order.
template <typename I>
__global__ void __launch_bounds__(1024) moe_route_kernel(const I* __restrict__ idx, int n, int capacity,
                                                         int* __restrict__ slot, int* __restrict__ count) {
  __shared__ int warp_tot[32];
  __shared__ int base;
  const int e = blockIdx.x;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  if (threadIdx.x == 0) base = 0;
  __syncthreads();
  for (int c0 = 0; c0 < n; c0 += blockDim.x) {
    const int i = c0 + threadIdx.x;
    const bool mine = i < n && (int)idx[i] == e;
    const unsigned b = __ballot_sync(0xffffffffu, mine);
    const int before = __popc(b & ((1u << lane) - 1));
    if (lane == 0) warp_tot[w] = __popc(b);
    __syncthreads();
    int off = base;
    for (int k = 0; k < w; ++k) off += warp_tot[k];
    if (mine) {
      const int pos = off + before;
      slot[i] = pos < capacity ? pos : -1;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int t = 0;
      for (int k = 0; k < (int)(blockDim.x >> 5); ++k) t += warp_tot[k];
      base += t;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) count[e] = base < capacity ? base : capacity;
}

// One warp per entry: copy (and optionally scale) one row of H bf16 into the owner's expert buffer.
template <typename I>
__global__ void __launch_bounds__(256)
moe_scatter_kernel(MoePeers pr, const __nv_bfloat16* __restrict__ src, long long ld_src, const I* __restrict__ idx,
                   const int* __restrict__ slot, const float* __restrict__ w, const int* __restrict__ count, int n,
                   int topk, int H, int e_local, int capacity, int num_experts) {
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  for (int i = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; i < n; i += warps) {
    const int s = slot[i];
    if (s < 0) continue;
    const int e = (int)idx[i];
    const int owner = e / e_local, el = e - owner * e_local;
    const __nv_bfloat16* row = src + (long long)(i / topk) * ld_src;
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(pr.buf[owner]) +
                         (((long long)el * pr.world + pr.rank) * capacity + s) * H;
    const float scale = w ? w[i] : 1.f;
    for (int c = lane * 8; c < H; c += 256) {
      uint4 u = *reinterpret_cast<const uint4*>(row + c);
      if (w) {
        float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), cc = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
        u.x = pack_bf16x2(a.x * scale, a.y * scale); u.y = pack_bf16x2(b.x * scale, b.y * scale);
        u.z = pack_bf16x2(cc.x * scale, cc.y * scale); u.w = pack_bf16x2(d.x * scale, d.y * scale);
      }
      *reinterpret_cast<uint4*>(dst + c) = u;
    }
  }
  // counts of this source rank, into every owner's table
  if (blockIdx.x == 0) {
    for (int e = threadIdx.x; e < num_experts; e += blockDim.x) {
      const int owner = e / e_local, el = e - owner * e_local;
      pr.counts[owner][el * pr.world + pr.rank] = count[e];
    }
  }
  // the block that finishes last publishes everything: ARRIVE(seq) in every rank's pad
  __shared__ int last;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned int prev = atomicAdd(pr.counter, 1u);
    last = prev == gridDim.x - 1;
    if (last) {
      *pr.counter = 0;
      __threadfence();
    }
  }
  __syncthreads();
  if (last && (int)threadIdx.x < pr.world) {
    __threadfence_system();
    st_release_sys(pr.pad[threadIdx.x] + pr.rank, pr.seq);   // channel ARRIVE = slots 0..7
  }
}

// Zero the slots [count, capacity) of every group of the local expert buffer. grid = (blocks, groups).
__global__ void __launch_bounds__(256)
moe_zero_tail_kernel(__nv_bfloat16* __restrict__ buf, const int* __restrict__ counts, int capacity, int H) {
  const int g = blockIdx.y;
  const int c = counts[g];
  const long long n16 = (long long)(capacity - c) * H / 8;
  uint4* p = reinterpret_cast<uint4*>(buf + ((long long)g * capacity + c) * H);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n16; i += (long long)gridDim.x * blockDim.x)
    p[i] = make_uint4(0u, 0u, 0u, 0u);
}

// One warp per token: out[t] = sum_j w[i] * row(i); optional dw[i] = <g[t], row(i)>.
template <typename I>
__global__ void __launch_bounds__(256)
moe_gather_kernel(MoePeers pr, __nv_bfloat16* __restrict__ out, long long ld_out, const I* __restrict__ idx,
                  const int* __restrict__ slot, const float* __restrict__ w, const __nv_bfloat16* __restrict__ g,
                  long long ld_g, float* __restrict__ dw, int T, int topk, int H, int e_local, int capacity,
                  int* status) {
  // every rank's expert outputs are in place? (ARRIVE channel of the buffer's pad, bounded wait)
  {
    int bad = 0;
    if ((int)threadIdx.x < pr.world) {
      const uint32_t* sl = pr.pad[pr.rank] + threadIdx.x;
      const unsigned long long limit = g_moe_wait_ns;
      const uint64_t t0 = globaltimer_ns();
      while ((int)(ld_acquire_sys(sl) - pr.seq) < 0) {
        if (globaltimer_ns() - t0 > limit) {
          bad = 1;
          if (status) atomicCAS(status, 0, (int)ATB_ERR_PEER_TIMEOUT);
          break;
        }
        __nanosleep(100);
      }
    }
    if (__syncthreads_or(bad)) return;
  }
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  constexpr int MAXK = 8;
  for (int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; t < T; t += warps) {
    float dots[MAXK];
#pragma unroll
    for (int j = 0; j < MAXK; ++j) dots[j] = 0.f;
    for (int c = lane * 8; c < H; c += 256) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      float gv[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (dw) {
        const uint4 u = *reinterpret_cast<const uint4*>(g + (long long)t * ld_g + c);
        const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), cc = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
        gv[0] = a.x; gv[1] = a.y; gv[2] = b.x; gv[3] = b.y; gv[4] = cc.x; gv[5] = cc.y; gv[6] = d.x; gv[7] = d.y;
      }
#pragma unroll
      for (int j = 0; j < MAXK; ++j) {
        if (j >= topk) break;
        const int i = t * topk + j;
        const int s = slot[i];
        if (s < 0) continue;
        const int e = (int)idx[i];
        const int owner = e / e_local, el = e - owner * e_local;
        const __nv_bfloat16* row = reinterpret_cast<const __nv_bfloat16*>(pr.buf[owner]) +
                                   (((long long)el * pr.world + pr.rank) * capacity + s) * H;
        const uint4 u = *reinterpret_cast<const uint4*>(row + c);
        const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), cc = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
        const float v[8] = {a.x, a.y, b.x, b.y, cc.x, cc.y, d.x, d.y};
        const float wj = w ? w[i] : 1.f;
#pragma unroll
        for (int q = 0; q < 8; ++q) acc[q] += wj * v[q];
        if (dw) {
#pragma unroll
          for (int q = 0; q < 8; ++q) dots[j] += gv[q] * v[q];
        }
      }
      if (out) {
        uint4 o;
        o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
        o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
        *reinterpret_cast<uint4*>(out + (long long)t * ld_out + c) = o;
      }
    }
    if (dw) {
#pragma unroll
      for (int j = 0; j < MAXK; ++j) {
        if (j >= topk) break;
        const float d = warp_sum(dots[j]);
        if (lane == 0) dw[t * topk + j] = d;      // 0 for dropped entries (nothing was accumulated)
      }
    }
  }
  // the block that finishes last tells the peers that this rank no longer reads their buffers (DONE)
  __shared__ int last;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int prev = atomicAdd(pr.counter, 1u);
    last = prev == gridDim.x - 1;
    if (last) {
      *pr.counter = 0;
      __threadfence();
    }
  }
  __syncthreads();
  if (last && (int)threadIdx.x < pr.world) {
    __threadfence_system();
    st_release_sys(pr.pad[threadIdx.x] + 16 + pr.rank, pr.seq);   // channel DONE = slots 16..23
  }
}

bool fill(MoePeers& pr, const unsigned long long* buf_ptrs, const unsigned long long* count_ptrs,
          const unsigned long long* pad_ptrs, void* counter, int rank, int world, unsigned int seq) {
  if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world) return false;
  for (int i = 0; i < MAX_RANKS; ++i) {
    pr.buf[i] = i < world ? reinterpret_cast<void*>(buf_ptrs[i]) : nullptr;
    pr.counts[i] = i < world && count_ptrs ? reinterpret_cast<int*>(count_ptrs[i]) : nullptr;
    pr.pad[i] = i < world ? reinterpret_cast<uint32_t*>(pad_ptrs[i]) : nullptr;
  }
  pr.counter = reinterpret_cast<unsigned int*>(counter);
  pr.rank = rank;
  pr.world = world;
  pr.seq = seq;
  return true;
}

int grid_for_warps(long long warps_needed, int cap_blocks) {
  long long g = (warps_needed + 7) / 8;
  if (g > cap_blocks) g = cap_blocks;
  return (int)(g < 1 ? 1 : g);
}
}  // namespace

extern "C" int atb_moe_set_wait_ns(unsigned long long ns) {
  return cudaMemcpyToSymbol(g_moe_wait_ns, &ns, sizeof(ns)) == cudaSuccess ? 0 : -5;
}

// idx: int64 (idx_i64 != 0) or int32 expert ids of n = T * k entries; slot[n], count[num_experts] int32 out.
extern "C" int atb_moe_route(const void* idx, int idx_i64, int n, int num_experts, int capacity, int* slot, int* count,
                             void* stream) {
  if (n <= 0 || num_experts <= 0 || capacity <= 0) return -1;
  cudaStream_t st = (cudaStream_t)stream;
  if (idx_i64) moe_route_kernel<long long><<<num_experts, 1024, 0, st>>>((const long long*)idx, n, capacity, slot, count);
  else moe_route_kernel<int><<<num_experts, 1024, 0, st>>>((const int*)idx, n, capacity, slot, count);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// src[T, H] bf16 (row pitch ld_src) -> peers' expert buffers. w (fp32 [n]) optional row scale.
// buf_ptrs / count_ptrs / pad_ptrs: `world` device addresses each. seq: use number of the buffer.
extern "C" int atb_moe_scatter(const unsigned long long* buf_ptrs, const unsigned long long* count_ptrs,
                               const unsigned long long* pad_ptrs, void* counter, int rank, int world, unsigned int seq,
                               const void* src, long long ld_src, const void* idx, int idx_i64, const int* slot,
                               const float* w, const int* count, int n, int topk, int H, int e_local, int capacity,
                               int num_experts, int max_blocks, void* stream) {
  MoePeers pr;
  if (!fill(pr, buf_ptrs, count_ptrs, pad_ptrs, counter, rank, world, seq)) return -1;
  if ((H & 7) || (ld_src & 7) || n <= 0 || topk <= 0 || e_local <= 0 || num_experts != e_local * world) return -1;
  const int grid = grid_for_warps(n, max_blocks > 0 ? max_blocks : 148 * 4);
  cudaStream_t st = (cudaStream_t)stream;
  if (idx_i64)
    moe_scatter_kernel<long long><<<grid, 256, 0, st>>>(pr, (const __nv_bfloat16*)src, ld_src, (const long long*)idx,
                                                         slot, w, count, n, topk, H, e_local, capacity, num_experts);
  else
    moe_scatter_kernel<int><<<grid, 256, 0, st>>>(pr, (const __nv_bfloat16*)src, ld_src, (const int*)idx, slot, w,
                                                   count, n, topk, H, e_local, capacity, num_experts);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// buf: local expert buffer [groups, capacity, H] bf16; counts: local int32 [groups].
extern "C" int atb_moe_zero_tail(void* buf, const int* counts, int groups, int capacity, int H, void* stream) {
  if (groups <= 0) return 0;
  if (H & 7) return -1;
  dim3 grid(32, groups);
  moe_zero_tail_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)buf, counts, capacity, H);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// out[T, H] bf16 = sum_j w[i] * peer rows. With dw != null also dw[i] = <g[t], row(i)> (g: [T, H] bf16).
// Waits (bounded) until every rank has signalled ARRIVE(seq) on this buffer's pad; signals DONE(seq).
extern "C" int atb_moe_gather(const unsigned long long* buf_ptrs, const unsigned long long* pad_ptrs, void* counter,
                              int rank, int world, unsigned int seq, void* out, long long ld_out, const void* idx,
                              int idx_i64, const int* slot, const float* w, const void* g, long long ld_g, float* dw,
                              int T, int topk, int H, int e_local, int capacity, int max_blocks, void* stream,
                              int* status) {
  MoePeers pr;
  if (!fill(pr, buf_ptrs, nullptr, pad_ptrs, counter, rank, world, seq)) return -1;
  if ((H & 7) || (ld_out & 7) || T <= 0 || topk <= 0 || topk > 8 || e_local <= 0 || (dw && (!g || (ld_g & 7))))
    return -1;
  const int grid = grid_for_warps(T, max_blocks > 0 ? max_blocks : 148 * 4);
  cudaStream_t st = (cudaStream_t)stream;
  if (idx_i64)
    moe_gather_kernel<long long><<<grid, 256, 0, st>>>(pr, (__nv_bfloat16*)out, ld_out, (const long long*)idx, slot, w,
                                                        (const __nv_bfloat16*)g, ld_g, dw, T, topk, H, e_local,
                                                        capacity, status);
  else
    moe_gather_kernel<int><<<grid, 256, 0, st>>>(pr, (__nv_bfloat16*)out, ld_out, (const int*)idx, slot, w,
                                                  (const __nv_bfloat16*)g, ld_g, dw, T, topk, H, e_local, capacity,
                                                  status);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
