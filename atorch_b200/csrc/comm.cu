// Fused collective + compute kernels over NVLink peer memory (symmetric buffers) for sm_100a.
//
// Every rank maps every peer's copy of a *symmetric* buffer (same size, same layout), a small signal
// pad per buffer, and - where the system offers NVLink SHARP - a multicast address of the buffer.
// The kernels read peers' data inside the kernel that does the arithmetic, either with plain 16-byte
// peer loads (ld.global over NVLink / NVSwitch, several in flight per thread: one peer load takes
// about 3 us, so bandwidth is bytes in flight / 3 us) or with multimem.ld_reduce, where the switch
// adds the ranks' values and one load returns the sum:
//
//   atb_p2p_reduce_scatter     out[slice] (+)= scale * sum_r grad_r[slice]
//   atb_p2p_rs_adamw           the same reduction feeding the sharded AdamW update in registers
//                              (master / m / v / bf16 working shard written by the same kernel)
//   atb_p2p_allreduce          in-place all-reduce (two-shot peer pulls, or one-shot multimem)
//   atb_p2p_allreduce_nesterov local-SGD outer step: mean of the replicas' parameters, Nesterov
//                              update of this rank's slice of the synchronised weights, new
//                              weights pulled back into every replica's parameter buffer
//   atb_p2p_allgather          pull all peers' shards into a local full buffer
//   atb_pad_signal / atb_pad_wait   stream-ordered cross-rank flags for everything else (the
//                              all-gather of the sharded engine runs on the copy engines)
//
// Cross-rank ordering uses sequence numbers in the signal pads (uint32[64] per buffer; the host
// counts the uses of a buffer and passes the number in). Channels of 8 slots each:
//   ARRIVE  rank r stores seq into slot r of every peer's pad when its input is in place
//   MID     ... when its reduced slice is in place (two-shot kernels only)
//   DONE    ... when it has finished reading the peers' buffers
//   READY   free for the host side (e.g. "parameters of step t are in place")
// A block that needs a condition polls its own pad with ld.acquire.sys; no block ever waits for
// another block of its own grid, so nothing here assumes that a whole grid is resident at once
// (two-shot kernels wait for the peers' grids and therefore clamp their grid to the SM count).
// The DONE signal is sent by whichever block finishes last (a counter that the block resets);
// nobody waits for it inside the kernel: the owner of a buffer waits for it (atb_pad_wait) before
// writing into the buffer again. Every wait is bounded (atb_set_comm_wait_ns, default 2 s): on
// timeout the kernel writes ATB_ERR_PEER_TIMEOUT to the status word, skips its remaining work and
// returns; since conditions are "slot >= seq", a later launch finds a consistent state again.
//
// These replace NCCL reduce_scatter / all_reduce + separate optimizer kernels on the hot paths of
// the reference (FSDP `_reduce_grad` + torch AdamW; atorch/local_sgd/FSDP/core/_runtime_utils.py:87-188;
// atorch/local_sgd/DDP/outer_optim_model_averager.py:109-194).
#include "common.cuh"

namespace {
using namespace atb;

constexpr int MAX_RANKS = 8;
constexpr int CH_ARRIVE = 0, CH_MID = 8, CH_DONE = 16, CH_READY = 24;
constexpr int THREADS = 256;  // x <= 128 registers: a block fits beside a resident GEMM CTA on the same SM
constexpr int UNROLL = 4;  // 16-byte peer loads in flight per thread

__device__ unsigned long long g_comm_wait_ns = ATB_WAIT_LIMIT_NS;

struct Peers {
  void* data[MAX_RANKS];      // peer copies of the symmetric data buffer
  uint32_t* pad[MAX_RANKS];   // peer signal pads
  void* mc;                   // multicast address of the buffer (nullptr: not available)
  unsigned int* counter;      // device word of this buffer: blocks finished (self-resetting)
  int rank, world;
  unsigned int seq;           // sequence number of this use of the buffer
};

ATB_DEVICE void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
ATB_DEVICE uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Tell every rank (slot `rank` of channel `ch` in each pad) that this rank reached `seq`.
// Called by one whole block after a __syncthreads(); the writes of that block (and, through the
// counter, of every block that finished before) are made visible first.
ATB_DEVICE void signal_all(const Peers& pr, int ch) {
  if ((int)threadIdx.x < pr.world) {
    __threadfence_system();
    st_release_sys(pr.pad[threadIdx.x] + ch + pr.rank, pr.seq);
  }
}

// Every rank has signalled `seq` on channel `ch`? Polled by the first `world` threads of the block;
// the outcome is shared by the whole block. Returns false when the wait ran out.
ATB_DEVICE bool wait_all(const Peers& pr, int ch, int* status) {
  int bad = 0;
  if ((int)threadIdx.x < pr.world) {
    const uint32_t* slot = pr.pad[pr.rank] + ch + threadIdx.x;
    const unsigned long long limit = g_comm_wait_ns;
    const uint64_t t0 = globaltimer_ns();
    // wrap-safe "slot >= seq"
    while ((int)(ld_acquire_sys(slot) - pr.seq) < 0) {
      if (globaltimer_ns() - t0 > limit) {
        bad = 1;
        if (status) atomicCAS(status, 0, (int)ATB_ERR_PEER_TIMEOUT);
        break;
      }
      __nanosleep(100);
    }
  }
  return __syncthreads_or(bad) == 0;
}

// Counts this block as finished; true for the block that finishes last (which resets the counter).
ATB_DEVICE bool block_finished_last(const Peers& pr, unsigned int phase_blocks) {
  __shared__ int last;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int prev = atomicAdd(pr.counter, 1u);
    last = prev == phase_blocks - 1;
    if (last) {
      *pr.counter = 0;
      __threadfence();
    }
  }
  __syncthreads();
  return last != 0;
}

template <typename T>
struct Vec;  // 16 bytes of T as floats
template <>
struct Vec<float> {
  static constexpr int N = 4;
  static ATB_DEVICE void unpack(const uint4& u, float (&v)[4]) {
    v[0] = __uint_as_float(u.x); v[1] = __uint_as_float(u.y); v[2] = __uint_as_float(u.z); v[3] = __uint_as_float(u.w);
  }
  static ATB_DEVICE uint4 pack(const float (&v)[4]) {
    return make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]), __float_as_uint(v[3]));
  }
};
template <>
struct Vec<__nv_bfloat16> {
  static constexpr int N = 8;
  static ATB_DEVICE void unpack(const uint4& u, float (&v)[8]) {
    const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
  }
  static ATB_DEVICE uint4 pack(const float (&v)[8]) {
    return make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7]));
  }
};

// The switch adds the 16-byte vectors of all ranks at this multicast address (fp32 accumulation).
template <typename T>
ATB_DEVICE uint4 multimem_ld_reduce(const void* mc_addr);
template <>
ATB_DEVICE uint4 multimem_ld_reduce<__nv_bfloat16>(const void* mc_addr) {
  uint4 r;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(mc_addr)
               : "memory");
  return r;
}
template <>
ATB_DEVICE uint4 multimem_ld_reduce<float>(const void* mc_addr) {
  uint4 r;
  float a, b, c, d;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(a), "=f"(b), "=f"(c), "=f"(d)
               : "l"(mc_addr)
               : "memory");
  r = make_uint4(__float_as_uint(a), __float_as_uint(b), __float_as_uint(c), __float_as_uint(d));
  return r;
}
ATB_DEVICE void multimem_st(void* mc_addr, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr),
               "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)),
               "f"(__uint_as_float(v.w))
               : "memory");
}

// Sum over all ranks of UNROLL vectors starting at element index i[u] of the symmetric buffer
// (negative index = nothing). All world*UNROLL (or, with NVLS, UNROLL) loads are issued before
// the first add, the peers are visited from rank+1 on so that they are not all hit in one order.
template <typename T, bool NVLS>
ATB_DEVICE void reduce_vectors(const Peers& pr, const long long (&i)[UNROLL], float (&acc)[UNROLL][Vec<T>::N]) {
  constexpr int N = Vec<T>::N;
  if constexpr (NVLS) {
    uint4 raw[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u)
      if (i[u] >= 0) raw[u] = multimem_ld_reduce<T>(reinterpret_cast<const T*>(pr.mc) + i[u]);
#pragma unroll
    for (int u = 0; u < UNROLL; ++u)
      if (i[u] >= 0) Vec<T>::unpack(raw[u], acc[u]);
  } else {
#pragma unroll
    for (int u = 0; u < UNROLL; ++u)
#pragma unroll
      for (int j = 0; j < N; ++j) acc[u][j] = 0.f;
    for (int k = 0; k < pr.world; k += 2) {
      const int p0 = (pr.rank + 1 + k) % pr.world;
      const int p1 = (pr.rank + 2 + k) % pr.world;
      const bool two = k + 1 < pr.world;
      uint4 a[UNROLL], b[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        if (i[u] >= 0) {
          a[u] = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(pr.data[p0]) + i[u]);
          if (two) b[u] = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(pr.data[p1]) + i[u]);
        }
      }
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        if (i[u] >= 0) {
          float v[N];
          Vec<T>::unpack(a[u], v);
#pragma unroll
          for (int j = 0; j < N; ++j) acc[u][j] += v[j];
          if (two) {
            Vec<T>::unpack(b[u], v);
#pragma unroll
            for (int j = 0; j < N; ++j) acc[u][j] += v[j];
          }
        }
      }
    }
  }
}

// Grid-stride walk over `count` elements in steps of UNROLL vectors per thread.
template <int N, typename F>
ATB_DEVICE void for_each_vectors(long long count, F&& body) {
  const long long per_iter = (long long)gridDim.x * blockDim.x * N;
  const long long first = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * N;
  for (long long base = first; base < count; base += per_iter * UNROLL) {
    long long idx[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const long long e = base + u * per_iter;
      idx[u] = e < count ? e : -1;
    }
    body(idx);
  }
}

struct AdamW {
  float lr, beta1, beta2, eps, weight_decay, bc1, bc2, grad_scale;
};

// ---------------------------------------------------------------------------------------------
// reduce-scatter of a unit's gradients, optionally fused with the sharded AdamW step.
// The symmetric buffer holds each rank's full flat gradient of the unit (n elements, type G);
// this rank owns [rank * n/W, (rank+1) * n/W).
//   ADAM = false : out[slice] (+)= scale * sum            (fp32 gradient shard)
//   ADAM = true  : master/m/v/lp of the shard updated from the sum; grad_out (optional) gets it
// ---------------------------------------------------------------------------------------------
template <typename G, bool NVLS, bool ADAM>
__global__ void __launch_bounds__(THREADS)
p2p_reduce_scatter_kernel(Peers pr, long long n, float* __restrict__ out, float scale, int accumulate,
                          float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                          __nv_bfloat16* __restrict__ lp, AdamW a, int* status) {
  constexpr int N = Vec<G>::N;
  const long long slice = n / pr.world;
  const long long lo = slice * pr.rank;
  if (blockIdx.x == 0) signal_all(pr, CH_ARRIVE);     // stream order: my gradients are complete
  const bool ok = wait_all(pr, CH_ARRIVE, status);     // ... and so are everybody else's
  if (ok) {
    for_each_vectors<N>(slice, [&](const long long(&idx)[UNROLL]) {
      long long gi[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) gi[u] = idx[u] >= 0 ? lo + idx[u] : -1;
      float g[UNROLL][N];
      reduce_vectors<G, NVLS>(pr, gi, g);
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        if (idx[u] < 0) continue;
        const long long i = idx[u];
        if constexpr (!ADAM) {
#pragma unroll
          for (int q = 0; q < N / 4; ++q) {
            float4 o = make_float4(g[u][4 * q] * scale, g[u][4 * q + 1] * scale, g[u][4 * q + 2] * scale,
                                   g[u][4 * q + 3] * scale);
            if (accumulate) {
              const float4 old = *reinterpret_cast<const float4*>(out + i + 4 * q);
              o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
            }
            *reinterpret_cast<float4*>(out + i + 4 * q) = o;
          }
        } else {
          float pbuf[N], mbuf[N], vbuf[N];
#pragma unroll
          for (int q = 0; q < N / 4; ++q) {
            const float4 p4 = *reinterpret_cast<const float4*>(master + i + 4 * q);
            const float4 m4 = *reinterpret_cast<const float4*>(m + i + 4 * q);
            const float4 v4 = *reinterpret_cast<const float4*>(v + i + 4 * q);
            pbuf[4 * q] = p4.x; pbuf[4 * q + 1] = p4.y; pbuf[4 * q + 2] = p4.z; pbuf[4 * q + 3] = p4.w;
            mbuf[4 * q] = m4.x; mbuf[4 * q + 1] = m4.y; mbuf[4 * q + 2] = m4.z; mbuf[4 * q + 3] = m4.w;
            vbuf[4 * q] = v4.x; vbuf[4 * q + 1] = v4.y; vbuf[4 * q + 2] = v4.z; vbuf[4 * q + 3] = v4.w;
          }
#pragma unroll
          for (int j = 0; j < N; ++j) {
            const float gj = g[u][j] * a.grad_scale;
            g[u][j] = gj;
            float p = pbuf[j] * (1.f - a.lr * a.weight_decay);
            mbuf[j] = a.beta1 * mbuf[j] + (1.f - a.beta1) * gj;
            vbuf[j] = a.beta2 * vbuf[j] + (1.f - a.beta2) * gj * gj;
            p -= a.lr * (mbuf[j] / a.bc1) / (sqrtf(vbuf[j] / a.bc2) + a.eps);
            pbuf[j] = p;
          }
#pragma unroll
          for (int q = 0; q < N / 4; ++q) {
            *reinterpret_cast<float4*>(master + i + 4 * q) =
                make_float4(pbuf[4 * q], pbuf[4 * q + 1], pbuf[4 * q + 2], pbuf[4 * q + 3]);
            *reinterpret_cast<float4*>(m + i + 4 * q) =
                make_float4(mbuf[4 * q], mbuf[4 * q + 1], mbuf[4 * q + 2], mbuf[4 * q + 3]);
            *reinterpret_cast<float4*>(v + i + 4 * q) =
                make_float4(vbuf[4 * q], vbuf[4 * q + 1], vbuf[4 * q + 2], vbuf[4 * q + 3]);
            if (out)
              *reinterpret_cast<float4*>(out + i + 4 * q) =
                  make_float4(g[u][4 * q], g[u][4 * q + 1], g[u][4 * q + 2], g[u][4 * q + 3]);
          }
          if (lp) {
#pragma unroll
            for (int q = 0; q < N / 2; ++q)
              reinterpret_cast<uint32_t*>(lp + i)[q] = pack_bf16x2(pbuf[2 * q], pbuf[2 * q + 1]);
          }
        }
      }
    });
  }
  // the block that finishes last tells the peers that this rank no longer reads their buffers
  if (block_finished_last(pr, gridDim.x)) signal_all(pr, CH_DONE);
}

// ---------------------------------------------------------------------------------------------
// all-reduce (sum * scale), in place on the symmetric buffer; n = elements, multiple of VEC * world
//   NVLS : one shot - reduce my slice through the switch and store it to every rank (multimem.st)
//   else : two shot - reduce my slice from all peers into my copy, then pull the other slices
// ---------------------------------------------------------------------------------------------
template <typename T, bool NVLS>
__global__ void __launch_bounds__(THREADS) p2p_allreduce_kernel(Peers pr, long long n, float scale, int* status) {
  constexpr int N = Vec<T>::N;
  const long long slice = n / pr.world;
  const long long lo = slice * pr.rank;
  T* mine = reinterpret_cast<T*>(pr.data[pr.rank]);
  if (blockIdx.x == 0) signal_all(pr, CH_ARRIVE);
  bool ok = wait_all(pr, CH_ARRIVE, status);            // every rank's input is in place
  if (ok) {
    for_each_vectors<N>(slice, [&](const long long(&idx)[UNROLL]) {
      long long gi[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) gi[u] = idx[u] >= 0 ? lo + idx[u] : -1;
      float acc[UNROLL][N];
      reduce_vectors<T, NVLS>(pr, gi, acc);
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        if (idx[u] < 0) continue;
#pragma unroll
        for (int j = 0; j < N; ++j) acc[u][j] *= scale;
        const uint4 o = Vec<T>::pack(acc[u]);
        if constexpr (NVLS) multimem_st(reinterpret_cast<T*>(pr.mc) + gi[u], o);
        else *reinterpret_cast<uint4*>(mine + gi[u]) = o;
      }
    });
  }
  if (block_finished_last(pr, gridDim.x)) signal_all(pr, CH_MID);   // my slice is reduced (and, NVLS, stored)
  ok = wait_all(pr, CH_MID, status) && ok;                            // ... and so is everybody else's
  if constexpr (!NVLS) {
    if (ok) {
      for (int k = 1; k < pr.world; ++k) {
        const int p = (pr.rank + k) % pr.world;
        const T* src = reinterpret_cast<const T*>(pr.data[p]) + slice * p;
        T* dst = mine + slice * p;
        for_each_vectors<N>(slice, [&](const long long(&idx)[UNROLL]) {
          uint4 t[UNROLL];
#pragma unroll
          for (int u = 0; u < UNROLL; ++u)
            if (idx[u] >= 0) t[u] = *reinterpret_cast<const uint4*>(src + idx[u]);
#pragma unroll
          for (int u = 0; u < UNROLL; ++u)
            if (idx[u] >= 0) *reinterpret_cast<uint4*>(dst + idx[u]) = t[u];
        });
      }
    }
  }
  // second use of the block counter in this launch: it was reset by the last block of the first use
  // only after every block had passed it, and no block reaches this point before CH_MID arrived
  if (block_finished_last(pr, gridDim.x)) signal_all(pr, CH_DONE);
}

// ---------------------------------------------------------------------------------------------
// Local-SGD outer step. The symmetric buffer holds every replica's CURRENT parameters (fp32, n
// elements). This rank owns slice [lo, lo + n/W) of the outer state (synced weights, momentum):
//   g = synced - mean_r(param_r);  buf = mu*buf + g;  synced -= lr * (g + mu*buf | buf)
// then every rank pulls the new slices into its own parameter buffer.
// ---------------------------------------------------------------------------------------------
template <bool NVLS>
__global__ void __launch_bounds__(THREADS)
p2p_allreduce_nesterov_kernel(Peers pr, long long n, float* __restrict__ synced, float* __restrict__ buf, float lr,
                              float mu, int nesterov, int first, float clip_scale, int* status) {
  const long long slice = n / pr.world;
  const long long lo = slice * pr.rank;
  const float inv_w = 1.f / pr.world;
  float* mine = reinterpret_cast<float*>(pr.data[pr.rank]);
  if (blockIdx.x == 0) signal_all(pr, CH_ARRIVE);
  bool ok = wait_all(pr, CH_ARRIVE, status);
  if (ok) {
    for_each_vectors<4>(slice, [&](const long long(&idx)[UNROLL]) {
      long long gi[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) gi[u] = idx[u] >= 0 ? lo + idx[u] : -1;
      float mean[UNROLL][4];
      reduce_vectors<float, NVLS>(pr, gi, mean);
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        if (idx[u] < 0) continue;
        const long long i = idx[u];
        const float4 s4 = *reinterpret_cast<const float4*>(synced + i);
        const float4 b4 = *reinterpret_cast<const float4*>(buf + i);
        float s[4] = {s4.x, s4.y, s4.z, s4.w}, b[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float g = (s[j] - mean[u][j] * inv_w) * clip_scale;
          b[j] = first ? g : mu * b[j] + g;
          s[j] -= lr * (nesterov ? g + mu * b[j] : b[j]);
        }
        const float4 ns = make_float4(s[0], s[1], s[2], s[3]);
        *reinterpret_cast<float4*>(synced + i) = ns;
        *reinterpret_cast<float4*>(buf + i) = make_float4(b[0], b[1], b[2], b[3]);
        if constexpr (NVLS)   // new weights straight into every replica's buffer
          multimem_st(reinterpret_cast<float*>(pr.mc) + lo + i, make_uint4(__float_as_uint(s[0]), __float_as_uint(s[1]),
                                                                          __float_as_uint(s[2]), __float_as_uint(s[3])));
        else                  // staged in my own copy; peers pull it after the next rendezvous
          *reinterpret_cast<float4*>(mine + lo + i) = ns;
      }
    });
  }
  if (block_finished_last(pr, gridDim.x)) signal_all(pr, CH_MID);
  ok = wait_all(pr, CH_MID, status) && ok;
  if constexpr (!NVLS) {
    if (ok) {
      for (int k = 1; k < pr.world; ++k) {
        const int p = (pr.rank + k) % pr.world;
        const float* src = reinterpret_cast<const float*>(pr.data[p]) + slice * p;
        float* dst = mine + slice * p;
        for_each_vectors<4>(slice, [&](const long long(&idx)[UNROLL]) {
          uint4 t[UNROLL];
#pragma unroll
          for (int u = 0; u < UNROLL; ++u)
            if (idx[u] >= 0) t[u] = *reinterpret_cast<const uint4*>(src + idx[u]);
#pragma unroll
          for (int u = 0; u < UNROLL; ++u)
            if (idx[u] >= 0) *reinterpret_cast<uint4*>(dst + idx[u]) = t[u];
        });
      }
    }
  }
  if (block_finished_last(pr, gridDim.x)) signal_all(pr, CH_DONE);
}

// all-gather: out[p * shard .. (p+1) * shard) = peer p's symmetric shard buffer (16-byte units)
__global__ void __launch_bounds__(THREADS)
p2p_allgather_kernel(Peers pr, long long shard_vec16, uint4* __restrict__ out, int* status) {
  if (blockIdx.x == 0) signal_all(pr, CH_ARRIVE);
  const bool ok = wait_all(pr, CH_ARRIVE, status);
  if (ok) {
    for (int k = 0; k < pr.world; ++k) {
      const int p = (pr.rank + 1 + k) % pr.world;
      const uint4* src = reinterpret_cast<const uint4*>(pr.data[p]);
      uint4* dst = out + shard_vec16 * p;
      for_each_vectors<1>(shard_vec16, [&](const long long(&idx)[UNROLL]) {
        uint4 t[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u)
          if (idx[u] >= 0) t[u] = src[idx[u]];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u)
          if (idx[u] >= 0) dst[idx[u]] = t[u];
      });
    }
  }
  if (block_finished_last(pr, gridDim.x)) signal_all(pr, CH_DONE);
}

// Stream-ordered flags: one block.
// dst[i] += src[i] for a bf16 source in this GPU's memory and an fp32 destination that may live on a peer (its
// address in the symmetric buffer): vector red.add through NVLink, no read of the destination. n % 8 == 0.
__global__ void peer_add_bf16_kernel(float* __restrict__ dst, const __nv_bfloat16* __restrict__ src, long long n8) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    const uint4 u = reinterpret_cast<const uint4*>(src)[i];
    const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
    float* o = dst + i * 8;
    asm volatile("red.relaxed.sys.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(o), "f"(a.x), "f"(a.y), "f"(b.x),
                 "f"(b.y)
                 : "memory");
    asm volatile("red.relaxed.sys.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(o + 4), "f"(c.x), "f"(c.y), "f"(d.x),
                 "f"(d.y)
                 : "memory");
  }
}

__global__ void pad_signal_kernel(Peers pr, int ch) {
  __syncthreads();
  signal_all(pr, ch);
}
__global__ void pad_wait_kernel(Peers pr, int ch, int* status) { wait_all(pr, ch, status); }

bool fill_peers(Peers& pr, const unsigned long long* data_ptrs, const unsigned long long* pad_ptrs,
                unsigned long long mc_ptr, void* counter, int rank, int world, unsigned int seq) {
  if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world) return false;
  for (int i = 0; i < MAX_RANKS; ++i) {
    pr.data[i] = i < world && data_ptrs ? reinterpret_cast<void*>(data_ptrs[i]) : nullptr;
    pr.pad[i] = i < world ? reinterpret_cast<uint32_t*>(pad_ptrs[i]) : nullptr;
  }
  pr.mc = reinterpret_cast<void*>(mc_ptr);
  pr.counter = reinterpret_cast<unsigned int*>(counter);
  pr.rank = rank;
  pr.world = world;
  pr.seq = seq;
  return true;
}

int sm_count() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  return sms;
}

// Two-shot kernels wait for the peers' grids: never launch more blocks than the GPU has SMs.
int grid_blocks(int max_blocks) {
  const int sms = sm_count();
  int g = max_blocks > 0 ? max_blocks : sms;
  if (g > sms) g = sms;
  return g < 1 ? 1 : g;
}

}  // namespace

// Upper bound of every cross-rank wait in this file, in nanoseconds (default 2 s). Tests of the
// failure path shorten it; takes effect for kernels launched afterwards on the current device.
extern "C" int atb_set_comm_wait_ns(unsigned long long ns) {
  return cudaMemcpyToSymbol(g_comm_wait_ns, &ns, sizeof(ns)) == cudaSuccess ? 0 : -5;
}

// Common arguments: `data_ptrs` / `pad_ptrs` host arrays of `world` device addresses (peer mappings
// of the symmetric buffer and of its signal pad, uint32[64], zeroed once); `mc_ptr` multicast address
// of the buffer or 0; `counter` one zero-initialised device uint32 per buffer; `seq` = number of this
// use of the buffer (1, 2, ...; the same on every rank). dtype: 0 bf16, 2 fp32. n must be a multiple
// of world * (16 / element size). `max_blocks` caps the grid (0 = one block per SM). use_nvls != 0
// takes the multimem path (needs mc_ptr).
extern "C" int atb_p2p_allreduce(const unsigned long long* data_ptrs, const unsigned long long* pad_ptrs,
                                 unsigned long long mc_ptr, void* counter, int rank, int world, unsigned int seq,
                                 long long n, long long offset, float scale, int dtype, int use_nvls, int max_blocks,
                                 void* stream, int* status) {
  Peers pr;
  if (!fill_peers(pr, data_ptrs, pad_ptrs, mc_ptr, counter, rank, world, seq)) return -1;
  const int vec = dtype == 0 ? 8 : 4;
  if (n % ((long long)world * vec) || offset < 0 || offset % vec) return -1;
  if (use_nvls && !mc_ptr) return -1;
  // `offset` (elements): the all-reduce covers [offset, offset + n) of the symmetric buffer
  const long long off_bytes = offset * (dtype == 0 ? 2 : 4);
  for (int i = 0; i < world; ++i) pr.data[i] = static_cast<char*>(pr.data[i]) + off_bytes;
  if (pr.mc) pr.mc = static_cast<char*>(pr.mc) + off_bytes;
  const int g = grid_blocks(max_blocks);
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == 0) {
    if (use_nvls) p2p_allreduce_kernel<__nv_bfloat16, true><<<g, THREADS, 0, st>>>(pr, n, scale, status);
    else p2p_allreduce_kernel<__nv_bfloat16, false><<<g, THREADS, 0, st>>>(pr, n, scale, status);
  } else if (dtype == 2) {
    if (use_nvls) p2p_allreduce_kernel<float, true><<<g, THREADS, 0, st>>>(pr, n, scale, status);
    else p2p_allreduce_kernel<float, false><<<g, THREADS, 0, st>>>(pr, n, scale, status);
  } else return -1;
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

extern "C" int atb_p2p_rs_adamw(const unsigned long long* data_ptrs, const unsigned long long* pad_ptrs,
                                unsigned long long mc_ptr, void* counter, int rank, int world, unsigned int seq,
                                long long n, float* master, float* m, float* v, void* lp, float* grad_out, float lr,
                                float beta1, float beta2, float eps, float weight_decay, int step, float grad_scale,
                                int grad_dtype, int use_nvls, int max_blocks, void* stream, int* status) {
  Peers pr;
  if (!fill_peers(pr, data_ptrs, pad_ptrs, mc_ptr, counter, rank, world, seq)) return -1;
  const int vec = grad_dtype == 0 ? 8 : 4;
  if (n % ((long long)world * vec)) return -1;
  if (use_nvls && !mc_ptr) return -1;
  AdamW a{lr, beta1, beta2, eps, weight_decay, 1.f - powf(beta1, (float)step), 1.f - powf(beta2, (float)step),
          grad_scale};
  const int g = grid_blocks(max_blocks);
  cudaStream_t st = (cudaStream_t)stream;
#define ATB_RS(G_, NV_)                                                                                            \
  p2p_reduce_scatter_kernel<G_, NV_, true><<<g, THREADS, 0, st>>>(pr, n, grad_out, 1.f, 0, master, m, v,          \
                                                                  (__nv_bfloat16*)lp, a, status)
  if (grad_dtype == 0) { if (use_nvls) ATB_RS(__nv_bfloat16, true); else ATB_RS(__nv_bfloat16, false); }
  else if (grad_dtype == 2) { if (use_nvls) ATB_RS(float, true); else ATB_RS(float, false); }
  else return -1;
#undef ATB_RS
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

extern "C" int atb_p2p_reduce_scatter(const unsigned long long* data_ptrs, const unsigned long long* pad_ptrs,
                                      unsigned long long mc_ptr, void* counter, int rank, int world, unsigned int seq,
                                      long long n, float* out, float scale, int accumulate, int grad_dtype,
                                      int use_nvls, int max_blocks, void* stream, int* status) {
  Peers pr;
  if (!fill_peers(pr, data_ptrs, pad_ptrs, mc_ptr, counter, rank, world, seq)) return -1;
  const int vec = grad_dtype == 0 ? 8 : 4;
  if (n % ((long long)world * vec)) return -1;
  if (use_nvls && !mc_ptr) return -1;
  const int g = grid_blocks(max_blocks);
  cudaStream_t st = (cudaStream_t)stream;
  AdamW a{};
#define ATB_RS(G_, NV_)                                                                                            \
  p2p_reduce_scatter_kernel<G_, NV_, false><<<g, THREADS, 0, st>>>(pr, n, out, scale, accumulate, nullptr, nullptr, \
                                                                   nullptr, nullptr, a, status)
  if (grad_dtype == 0) { if (use_nvls) ATB_RS(__nv_bfloat16, true); else ATB_RS(__nv_bfloat16, false); }
  else if (grad_dtype == 2) { if (use_nvls) ATB_RS(float, true); else ATB_RS(float, false); }
  else return -1;
#undef ATB_RS
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

extern "C" int atb_p2p_allreduce_nesterov(const unsigned long long* data_ptrs, const unsigned long long* pad_ptrs,
                                          unsigned long long mc_ptr, void* counter, int rank, int world,
                                          unsigned int seq, long long n, float* synced, float* momentum_buf, float lr,
                                          float momentum, int nesterov, int first_step, float clip_scale,
                                          int use_nvls, int max_blocks, void* stream, int* status) {
  Peers pr;
  if (!fill_peers(pr, data_ptrs, pad_ptrs, mc_ptr, counter, rank, world, seq)) return -1;
  if (n % ((long long)world * 4)) return -1;
  if (use_nvls && !mc_ptr) return -1;
  const int g = grid_blocks(max_blocks);
  cudaStream_t st = (cudaStream_t)stream;
  if (use_nvls)
    p2p_allreduce_nesterov_kernel<true><<<g, THREADS, 0, st>>>(pr, n, synced, momentum_buf, lr, momentum, nesterov,
                                                               first_step, clip_scale, status);
  else
    p2p_allreduce_nesterov_kernel<false><<<g, THREADS, 0, st>>>(pr, n, synced, momentum_buf, lr, momentum, nesterov,
                                                                first_step, clip_scale, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

extern "C" int atb_p2p_allgather(const unsigned long long* data_ptrs, const unsigned long long* pad_ptrs,
                                 void* counter, int rank, int world, unsigned int seq, long long shard_bytes,
                                 void* out, int max_blocks, void* stream, int* status) {
  Peers pr;
  if (!fill_peers(pr, data_ptrs, pad_ptrs, 0, counter, rank, world, seq)) return -1;
  if (shard_bytes % 16) return -1;
  const int g = grid_blocks(max_blocks);
  p2p_allgather_kernel<<<g, THREADS, 0, (cudaStream_t)stream>>>(pr, shard_bytes / 16, (uint4*)out, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// channel: 0 arrive, 1 mid, 2 done, 3 ready. Signal = "this rank reached seq on that channel",
// wait = "every rank did" (bounded; a timeout lands in the status word).
extern "C" int atb_pad_signal(const unsigned long long* pad_ptrs, int rank, int world, unsigned int seq, int channel,
                              void* stream) {
  Peers pr;
  if (channel < 0 || channel > 3 || !fill_peers(pr, nullptr, pad_ptrs, 0, nullptr, rank, world, seq)) return -1;
  pad_signal_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(pr, channel * 8);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
extern "C" int atb_pad_wait(const unsigned long long* pad_ptrs, int rank, int world, unsigned int seq, int channel,
                            void* stream, int* status) {
  Peers pr;
  if (channel < 0 || channel > 3 || !fill_peers(pr, nullptr, pad_ptrs, 0, nullptr, rank, world, seq)) return -1;
  pad_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(pr, channel * 8, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// dst (fp32, this GPU's or a peer's address inside a symmetric buffer) += src (bf16, local). n % 8 == 0; both 16-byte
// aligned. Completion is ordered with the stream; pair it with a pad signal so that the owner knows when to read.
extern "C" int atb_peer_add_bf16(unsigned long long dst, const void* src, long long n, void* stream) {
  if (n <= 0) return 0;
  if ((n & 7) || (dst & 15) || (reinterpret_cast<uintptr_t>(src) & 15)) return -1;
  const long long n8 = n >> 3;
  long long g = (n8 + 255) / 256;
  if (g > 148 * 8) g = 148 * 8;
  peer_add_bf16_kernel<<<(unsigned)g, 256, 0, (cudaStream_t)stream>>>(reinterpret_cast<float*>(dst),
                                                                      (const __nv_bfloat16*)src, n8);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
