// Fused collective + compute kernels over NVLink peer memory (symmetric buffers) for sm_100a.
//
// Every rank maps every peer's copy of a *symmetric* buffer (same size, same layout) and of a small
// signal pad. The kernels below read peers' data with plain 16-byte peer loads (ld.global over
// NVLink / NVSwitch) inside the same kernel that does the arithmetic, so no gathered or reduced copy
// is ever materialised by a separate collective:
//
//   atb_p2p_allreduce          two-shot all-reduce in place (reduce my slice from all peers, then
//                              pull everybody's reduced slice)
//   atb_p2p_rs_adamw           gradient reduce-scatter fused with the sharded AdamW update: my slice of
//                              the unit's gradients is summed over the peers in registers and goes
//                              straight into master / m / v and the bf16 working shard
//   atb_p2p_allreduce_nesterov local-SGD outer step: pseudo-gradient slice reduced over the peers,
//                              Nesterov momentum update of this rank's slice of the synchronised
//                              weights (outer state is sharded 1/W per rank), new weights pushed back
//                              into every replica's parameter buffer
//   atb_p2p_allgather          pull all peers' shards into a local full buffer (baseline building block)
//
// Cross-rank ordering uses sequence numbers in the signal pads: rank r stores `seq` into slot r of
// every peer's pad (st.release.sys) and waits until all slots of its own pad reach `seq`
// (ld.acquire.sys). Every such wait is bounded (ATB_WAIT_LIMIT_NS); on timeout the kernel writes
// ATB_ERR_PEER_TIMEOUT to the status word, skips its remaining work and returns. Block 0 does the
// handshake and releases the other blocks of the grid through a device-scope flag, so blocks never
// wait for later blocks (no co-residency assumption).
//
// These replace NCCL reduce_scatter / all_reduce + separate optimizer kernels on the hot paths of
// the reference (FSDP `_reduce_grad` + torch AdamW; atorch/local_sgd/FSDP/core/_runtime_utils.py:87-188;
// atorch/local_sgd/DDP/outer_optim_model_averager.py:109-194).
#include "common.cuh"

namespace {
using namespace atb;

constexpr int MAX_RANKS = 8;

struct Peers {
  void* data[MAX_RANKS];      // peer copies of the symmetric data buffer
  uint32_t* pad[MAX_RANKS];   // peer signal pads: uint32[MAX_RANKS] per channel
  int rank, world;
};

// Device-resident bookkeeping of one symmetric buffer: sequence counter and intra-grid flags.
struct SyncState {
  unsigned int seq;        // last sequence number used on the signal pad
  unsigned int go;         // grid release flag (monotonic)
  unsigned int done;       // blocks that finished the current phase
  unsigned int failed;     // set when a cross-rank wait ran out
};

ATB_DEVICE void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
ATB_DEVICE uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
ATB_DEVICE void st_release_gpu(unsigned int* p, unsigned int v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
ATB_DEVICE unsigned int ld_acquire_gpu(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Grid-wide rendezvous with all peers. Called by every thread of every block. `phase` counts the
// barriers of this launch (0, 1, ...); `base` = sequence number before the launch.
// Returns false if a wait ran out (the whole grid then sees `failed`).
ATB_DEVICE bool cross_rank_barrier(const Peers& pr, SyncState* st, unsigned int base, unsigned int phase,
                                   unsigned int nblocks, int* status) {
  const unsigned int target = base + phase + 1;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();  // this block's global writes are visible before it reports in
    atomicAdd(&st->done, 1u);
  }
  if (blockIdx.x == 0) {
    // wait until every block of this grid has finished the previous phase
    if (threadIdx.x == 0) {
      const unsigned int need = nblocks * (phase + 1);
      const uint64_t t0 = globaltimer_ns();
      while (ld_acquire_gpu(&st->done) < need) {
        if (globaltimer_ns() - t0 > ATB_WAIT_LIMIT_NS) { st->failed = 1; break; }
        __nanosleep(64);
      }
      __threadfence_system();
    }
    __syncthreads();
    if ((int)threadIdx.x < pr.world) {
      st_release_sys(pr.pad[threadIdx.x] + pr.rank, target);
      const uint64_t t0 = globaltimer_ns();
      while (ld_acquire_sys(pr.pad[pr.rank] + threadIdx.x) < target) {
        if (globaltimer_ns() - t0 > ATB_WAIT_LIMIT_NS || st->failed) {
          st->failed = 1;
          if (status) atomicCAS(status, 0, (int)ATB_ERR_PEER_TIMEOUT);
          break;
        }
        __nanosleep(32);
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) st_release_gpu(&st->go, target);
  } else if (threadIdx.x == 0) {
    const uint64_t t0 = globaltimer_ns();
    while (ld_acquire_gpu(&st->go) < target) {
      if (globaltimer_ns() - t0 > 2 * ATB_WAIT_LIMIT_NS) {
        st->failed = 1;
        if (status) atomicCAS(status, 0, (int)ATB_ERR_PEER_TIMEOUT);
        break;
      }
      __nanosleep(64);
    }
  }
  __syncthreads();
  return *reinterpret_cast<volatile unsigned int*>(&st->failed) == 0;
}

// End-of-launch bookkeeping by the last block: publish the new sequence base, clear counters.
ATB_DEVICE void finish_launch(SyncState* st, unsigned int base, unsigned int nphases, unsigned int nblocks) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int prev = atomicAdd(&st->done, 1u);
    if (prev == nblocks * (nphases + 1) - 1) {
      st->done = 0;
      st->seq = base + nphases;
      __threadfence();
    }
  }
}

template <typename T>
ATB_DEVICE void load_vec(const T* p, float (&v)[16 / sizeof(T)]);
template <>
ATB_DEVICE void load_vec<float>(const float* p, float (&v)[4]) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
}
template <>
ATB_DEVICE void load_vec<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
}
template <typename T>
ATB_DEVICE void store_vec(T* p, const float (&v)[16 / sizeof(T)]);
template <>
ATB_DEVICE void store_vec<float>(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
template <>
ATB_DEVICE void store_vec<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 u;
  u.x = pack_bf16x2(v[0], v[1]); u.y = pack_bf16x2(v[2], v[3]);
  u.z = pack_bf16x2(v[4], v[5]); u.w = pack_bf16x2(v[6], v[7]);
  *reinterpret_cast<uint4*>(p) = u;
}

// Sum over all ranks of elements [i, i + VEC) of the symmetric buffer, starting with the local copy
// and going round the ring from rank+1 so that the peers are not all hit in the same order.
template <typename T>
ATB_DEVICE void reduce_peers(const Peers& pr, long long i, float (&acc)[16 / sizeof(T)]) {
  constexpr int VEC = 16 / sizeof(T);
#pragma unroll
  for (int j = 0; j < VEC; ++j) acc[j] = 0.f;
  for (int k = 0; k < pr.world; ++k) {
    const int p = (pr.rank + k) % pr.world;
    float v[VEC];
    load_vec<T>(reinterpret_cast<const T*>(pr.data[p]) + i, v);
#pragma unroll
    for (int j = 0; j < VEC; ++j) acc[j] += v[j];
  }
}

// ---------------------------------------------------------------------------------------------
// all-reduce (sum * scale), in place on the symmetric buffer; n = elements, multiple of VEC * world
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(512) p2p_allreduce_kernel(Peers pr, SyncState* st, long long n, float scale,
                                                            int* status) {
  constexpr int VEC = 16 / sizeof(T);
  const unsigned int base = st->seq;
  const long long slice = n / pr.world;
  const long long lo = slice * pr.rank;
  T* mine = reinterpret_cast<T*>(pr.data[pr.rank]);
  bool ok = cross_rank_barrier(pr, st, base, 0, gridDim.x, status);  // every rank's input is in place
  if (ok) {
    for (long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * VEC; i < slice;
         i += (long long)gridDim.x * blockDim.x * VEC) {
      float acc[VEC];
      reduce_peers<T>(pr, lo + i, acc);
#pragma unroll
      for (int j = 0; j < VEC; ++j) acc[j] *= scale;
      store_vec<T>(mine + lo + i, acc);
    }
  }
  ok = cross_rank_barrier(pr, st, base, 1, gridDim.x, status) && ok;  // all slices reduced
  if (ok) {
    for (int k = 1; k < pr.world; ++k) {
      const int p = (pr.rank + k) % pr.world;
      const T* src = reinterpret_cast<const T*>(pr.data[p]) + slice * p;
      T* dst = mine + slice * p;
      for (long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * VEC; i < slice;
           i += (long long)gridDim.x * blockDim.x * VEC)
        *reinterpret_cast<uint4*>(dst + i) = *reinterpret_cast<const uint4*>(src + i);
    }
  }
  cross_rank_barrier(pr, st, base, 2, gridDim.x, status);  // nobody still reads my slice
  finish_launch(st, base, 3, gridDim.x);
}

// ---------------------------------------------------------------------------------------------
// reduce-scatter of the unit gradients fused with the sharded AdamW step.
// The symmetric buffer holds each rank's full flat gradient of the unit (n elements, type G);
// this rank owns [rank * n/W, (rank+1) * n/W) and updates master/m/v/lp of that shard.
// ---------------------------------------------------------------------------------------------
struct AdamW {
  float lr, beta1, beta2, eps, weight_decay, bc1, bc2, grad_scale;
};

template <typename G>
__global__ void __launch_bounds__(512)
p2p_rs_adamw_kernel(Peers pr, SyncState* st, long long n, float* __restrict__ master, float* __restrict__ m,
                    float* __restrict__ v, __nv_bfloat16* __restrict__ lp, float* __restrict__ grad_out, AdamW a,
                    int* status) {
  constexpr int VEC = 16 / sizeof(G);
  const unsigned int base = st->seq;
  const long long slice = n / pr.world;
  const long long lo = slice * pr.rank;
  bool ok = cross_rank_barrier(pr, st, base, 0, gridDim.x, status);
  if (ok) {
    for (long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * VEC; i < slice;
         i += (long long)gridDim.x * blockDim.x * VEC) {
      float g[VEC];
      reduce_peers<G>(pr, lo + i, g);
      float pbuf[VEC], mbuf[VEC], vbuf[VEC];
#pragma unroll
      for (int q = 0; q < VEC / 4; ++q) {
        const float4 p4 = *reinterpret_cast<const float4*>(master + i + 4 * q);
        const float4 m4 = *reinterpret_cast<const float4*>(m + i + 4 * q);
        const float4 v4 = *reinterpret_cast<const float4*>(v + i + 4 * q);
        pbuf[4 * q] = p4.x; pbuf[4 * q + 1] = p4.y; pbuf[4 * q + 2] = p4.z; pbuf[4 * q + 3] = p4.w;
        mbuf[4 * q] = m4.x; mbuf[4 * q + 1] = m4.y; mbuf[4 * q + 2] = m4.z; mbuf[4 * q + 3] = m4.w;
        vbuf[4 * q] = v4.x; vbuf[4 * q + 1] = v4.y; vbuf[4 * q + 2] = v4.z; vbuf[4 * q + 3] = v4.w;
      }
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        const float gj = g[j] * a.grad_scale;
        g[j] = gj;
        float p = pbuf[j] * (1.f - a.lr * a.weight_decay);
        mbuf[j] = a.beta1 * mbuf[j] + (1.f - a.beta1) * gj;
        vbuf[j] = a.beta2 * vbuf[j] + (1.f - a.beta2) * gj * gj;
        p -= a.lr * (mbuf[j] / a.bc1) / (sqrtf(vbuf[j] / a.bc2) + a.eps);
        pbuf[j] = p;
      }
#pragma unroll
      for (int q = 0; q < VEC / 4; ++q) {
        *reinterpret_cast<float4*>(master + i + 4 * q) =
            make_float4(pbuf[4 * q], pbuf[4 * q + 1], pbuf[4 * q + 2], pbuf[4 * q + 3]);
        *reinterpret_cast<float4*>(m + i + 4 * q) =
            make_float4(mbuf[4 * q], mbuf[4 * q + 1], mbuf[4 * q + 2], mbuf[4 * q + 3]);
        *reinterpret_cast<float4*>(v + i + 4 * q) =
            make_float4(vbuf[4 * q], vbuf[4 * q + 1], vbuf[4 * q + 2], vbuf[4 * q + 3]);
        if (grad_out)
          *reinterpret_cast<float4*>(grad_out + i + 4 * q) = make_float4(g[4 * q], g[4 * q + 1], g[4 * q + 2], g[4 * q + 3]);
      }
      if (lp) {
#pragma unroll
        for (int q = 0; q < VEC / 2; ++q)
          reinterpret_cast<uint32_t*>(lp + i)[q] = pack_bf16x2(pbuf[2 * q], pbuf[2 * q + 1]);
      }
    }
  }
  cross_rank_barrier(pr, st, base, 1, gridDim.x, status);  // peers have finished reading my gradients
  finish_launch(st, base, 2, gridDim.x);
}

// Same reduce-scatter without the optimizer: out[slice] (+)= scale * sum_r grad_r[slice]  (fp32 out)
template <typename G>
__global__ void __launch_bounds__(512)
p2p_reduce_scatter_kernel(Peers pr, SyncState* st, long long n, float* __restrict__ out, float scale, int accumulate,
                          int* status) {
  constexpr int VEC = 16 / sizeof(G);
  const unsigned int base = st->seq;
  const long long slice = n / pr.world;
  const long long lo = slice * pr.rank;
  const bool ok = cross_rank_barrier(pr, st, base, 0, gridDim.x, status);
  if (ok) {
    for (long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * VEC; i < slice;
         i += (long long)gridDim.x * blockDim.x * VEC) {
      float g[VEC];
      reduce_peers<G>(pr, lo + i, g);
#pragma unroll
      for (int q = 0; q < VEC / 4; ++q) {
        float4 o = make_float4(g[4 * q] * scale, g[4 * q + 1] * scale, g[4 * q + 2] * scale, g[4 * q + 3] * scale);
        if (accumulate) {
          const float4 old = *reinterpret_cast<const float4*>(out + i + 4 * q);
          o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
        }
        *reinterpret_cast<float4*>(out + i + 4 * q) = o;
      }
    }
  }
  cross_rank_barrier(pr, st, base, 1, gridDim.x, status);
  finish_launch(st, base, 2, gridDim.x);
}

// ---------------------------------------------------------------------------------------------
// Local-SGD outer step. The symmetric buffer holds every replica's CURRENT parameters (fp32, n
// elements). This rank owns slice [lo, lo + n/W) of the outer state (synced weights, momentum):
//   g = synced - mean_r(param_r);  buf = mu*buf + g;  synced -= lr * (g + mu*buf | buf)
// then the new synced slice is written into every replica's parameter buffer (peer stores).
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(512)
p2p_allreduce_nesterov_kernel(Peers pr, SyncState* st, long long n, float* __restrict__ synced,
                              float* __restrict__ buf, float lr, float mu, int nesterov, int first, float clip_scale,
                              int* status) {
  const unsigned int base = st->seq;
  const long long slice = n / pr.world;
  const long long lo = slice * pr.rank;
  const float inv_w = 1.f / pr.world;
  bool ok = cross_rank_barrier(pr, st, base, 0, gridDim.x, status);
  if (ok) {
    for (long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 4; i < slice;
         i += (long long)gridDim.x * blockDim.x * 4) {
      float mean[4];
      reduce_peers<float>(pr, lo + i, mean);
      const float4 s4 = *reinterpret_cast<const float4*>(synced + i);
      const float4 b4 = *reinterpret_cast<const float4*>(buf + i);
      float s[4] = {s4.x, s4.y, s4.z, s4.w}, b[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float g = (s[j] - mean[j] * inv_w) * clip_scale;
        b[j] = first ? g : mu * b[j] + g;
        s[j] -= lr * (nesterov ? g + mu * b[j] : b[j]);
      }
      const float4 ns = make_float4(s[0], s[1], s[2], s[3]);
      *reinterpret_cast<float4*>(synced + i) = ns;
      *reinterpret_cast<float4*>(buf + i) = make_float4(b[0], b[1], b[2], b[3]);
      // stage the result in my own copy first; peers pull it after the next barrier
      *reinterpret_cast<float4*>(reinterpret_cast<float*>(pr.data[pr.rank]) + lo + i) = ns;
    }
  }
  ok = cross_rank_barrier(pr, st, base, 1, gridDim.x, status) && ok;
  if (ok) {
    float* mine = reinterpret_cast<float*>(pr.data[pr.rank]);
    for (int k = 1; k < pr.world; ++k) {
      const int p = (pr.rank + k) % pr.world;
      const float* src = reinterpret_cast<const float*>(pr.data[p]) + slice * p;
      float* dst = mine + slice * p;
      for (long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 4; i < slice;
           i += (long long)gridDim.x * blockDim.x * 4)
        *reinterpret_cast<float4*>(dst + i) = *reinterpret_cast<const float4*>(src + i);
    }
  }
  cross_rank_barrier(pr, st, base, 2, gridDim.x, status);
  finish_launch(st, base, 3, gridDim.x);
}

// all-gather: out[p * shard .. (p+1) * shard) = peer p's symmetric shard buffer (bytes, 16-byte units)
__global__ void __launch_bounds__(512)
p2p_allgather_kernel(Peers pr, SyncState* st, long long shard_vec16, uint4* __restrict__ out, int* status) {
  const unsigned int base = st->seq;
  const bool ok = cross_rank_barrier(pr, st, base, 0, gridDim.x, status);
  if (ok) {
    for (int k = 0; k < pr.world; ++k) {
      const int p = (pr.rank + k) % pr.world;
      const uint4* src = reinterpret_cast<const uint4*>(pr.data[p]);
      uint4* dst = out + shard_vec16 * p;
      for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < shard_vec16;
           i += (long long)gridDim.x * blockDim.x)
        dst[i] = src[i];
    }
  }
  cross_rank_barrier(pr, st, base, 1, gridDim.x, status);
  finish_launch(st, base, 2, gridDim.x);
}

bool fill_peers(Peers& pr, const unsigned long long* data_ptrs, const unsigned long long* pad_ptrs, int rank,
                int world) {
  if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world) return false;
  for (int i = 0; i < world; ++i) {
    pr.data[i] = reinterpret_cast<void*>(data_ptrs[i]);
    pr.pad[i] = reinterpret_cast<uint32_t*>(pad_ptrs[i]);
  }
  pr.rank = rank;
  pr.world = world;
  return true;
}

int grid_blocks(int max_blocks) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int g = max_blocks > 0 ? max_blocks : sms;
  return g < 1 ? 1 : g;
}

}  // namespace

// `data_ptrs` / `pad_ptrs`: host arrays of `world` device addresses (peer mappings of the symmetric
// buffer and of its signal pad, uint32[8], zero-initialised once). `sync_state`: 16-byte device
// struct per symmetric buffer, zero-initialised once. dtype: 0 bf16, 2 fp32. n must be a multiple
// of world * (16 / element size). `max_blocks` caps the grid (0 = one block per SM).
extern "C" int atb_p2p_allreduce(const unsigned long long* data_ptrs, const unsigned long long* pad_ptrs, int rank,
                                 int world, void* sync_state, long long n, float scale, int dtype, int max_blocks,
                                 void* stream, int* status) {
  Peers pr;
  if (!fill_peers(pr, data_ptrs, pad_ptrs, rank, world)) return -1;
  const int vec = dtype == 0 ? 8 : 4;
  if (n % ((long long)world * vec)) return -1;
  const int g = grid_blocks(max_blocks);
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == 0)
    p2p_allreduce_kernel<__nv_bfloat16><<<g, 512, 0, st>>>(pr, (SyncState*)sync_state, n, scale, status);
  else if (dtype == 2)
    p2p_allreduce_kernel<float><<<g, 512, 0, st>>>(pr, (SyncState*)sync_state, n, scale, status);
  else return -1;
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

extern "C" int atb_p2p_rs_adamw(const unsigned long long* data_ptrs, const unsigned long long* pad_ptrs, int rank,
                                int world, void* sync_state, long long n, float* master, float* m, float* v, void* lp,
                                float* grad_out, float lr, float beta1, float beta2, float eps, float weight_decay,
                                int step, float grad_scale, int grad_dtype, int max_blocks, void* stream,
                                int* status) {
  Peers pr;
  if (!fill_peers(pr, data_ptrs, pad_ptrs, rank, world)) return -1;
  const int vec = grad_dtype == 0 ? 8 : 4;
  if (n % ((long long)world * vec)) return -1;
  AdamW a{lr, beta1, beta2, eps, weight_decay, 1.f - powf(beta1, (float)step), 1.f - powf(beta2, (float)step),
          grad_scale};
  const int g = grid_blocks(max_blocks);
  cudaStream_t st = (cudaStream_t)stream;
  if (grad_dtype == 0)
    p2p_rs_adamw_kernel<__nv_bfloat16><<<g, 512, 0, st>>>(pr, (SyncState*)sync_state, n, master, m, v,
                                                          (__nv_bfloat16*)lp, grad_out, a, status);
  else if (grad_dtype == 2)
    p2p_rs_adamw_kernel<float><<<g, 512, 0, st>>>(pr, (SyncState*)sync_state, n, master, m, v, (__nv_bfloat16*)lp,
                                                  grad_out, a, status);
  else return -1;
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

extern "C" int atb_p2p_reduce_scatter(const unsigned long long* data_ptrs, const unsigned long long* pad_ptrs,
                                      int rank, int world, void* sync_state, long long n, float* out, float scale,
                                      int accumulate, int grad_dtype, int max_blocks, void* stream, int* status) {
  Peers pr;
  if (!fill_peers(pr, data_ptrs, pad_ptrs, rank, world)) return -1;
  const int vec = grad_dtype == 0 ? 8 : 4;
  if (n % ((long long)world * vec)) return -1;
  const int g = grid_blocks(max_blocks);
  cudaStream_t st = (cudaStream_t)stream;
  if (grad_dtype == 0)
    p2p_reduce_scatter_kernel<__nv_bfloat16><<<g, 512, 0, st>>>(pr, (SyncState*)sync_state, n, out, scale, accumulate,
                                                                status);
  else if (grad_dtype == 2)
    p2p_reduce_scatter_kernel<float><<<g, 512, 0, st>>>(pr, (SyncState*)sync_state, n, out, scale, accumulate, status);
  else return -1;
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

extern "C" int atb_p2p_allreduce_nesterov(const unsigned long long* data_ptrs, const unsigned long long* pad_ptrs,
                                          int rank, int world, void* sync_state, long long n, float* synced,
                                          float* momentum_buf, float lr, float momentum, int nesterov,
                                          int first_step, float clip_scale, int max_blocks, void* stream,
                                          int* status) {
  Peers pr;
  if (!fill_peers(pr, data_ptrs, pad_ptrs, rank, world)) return -1;
  if (n % ((long long)world * 4)) return -1;
  const int g = grid_blocks(max_blocks);
  p2p_allreduce_nesterov_kernel<<<g, 512, 0, (cudaStream_t)stream>>>(pr, (SyncState*)sync_state, n, synced,
                                                                    momentum_buf, lr, momentum, nesterov, first_step,
                                                                    clip_scale, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

extern "C" int atb_p2p_allgather(const unsigned long long* data_ptrs, const unsigned long long* pad_ptrs, int rank,
                                 int world, void* sync_state, long long shard_bytes, void* out, int max_blocks,
                                 void* stream, int* status) {
  Peers pr;
  if (!fill_peers(pr, data_ptrs, pad_ptrs, rank, world)) return -1;
  if (shard_bytes % 16) return -1;
  const int g = grid_blocks(max_blocks);
  p2p_allgather_kernel<<<g, 512, 0, (cudaStream_t)stream>>>(pr, (SyncState*)sync_state, shard_bytes / 16, (uint4*)out,
                                                           status);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
