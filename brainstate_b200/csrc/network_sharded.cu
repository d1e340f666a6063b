// Fused E/I network step for a postsynaptic shard: one launch per GPU for many steps,
// neuron state resident in shared memory, ONE grid-wide barrier per step, spikes
// exchanged between the GPUs of a node as compact id lists pushed over NVLink.
//
// The reference runs the network on one device (examples/400_CUBA_2005_bpu.py:60-66:
// two EventFixedProb products, Expon, CUBA/COBA, LIFRef per step); sharding by
// postsynaptic neuron has no counterpart there beyond the generic device-mesh
// precedent of brainstate/transform/_shard_map.py:96.
//
// Every rank owns a contiguous block of neurons and, of both projections, the
// synapses that target them (a CSR block: rows = presynaptic neurons of the whole
// network, columns = local neurons).  One 1024-thread block per SM owns a contiguous
// range of the rank's spike words.  A step of one block:
//
//   1. update its neurons (synapse decay + pending increment, membrane, threshold),
//      collecting the ones that spiked in a shared-memory list; a warp that finds spikes
//      stores their ids into every peer's inbox right away — 64-bit words
//      (tag << 32 | payload), tag = exchange sequence number + 1, so that every word
//      validates itself and neither a fence nor a separate flag is needed;
//   2. link warps (one per peer) complete the list with its header (the count) and then
//      poll their own inbox for the list the same block index of that peer pushed,
//      fetching the header and the first 31 ids in one round trip;
//   3. meanwhile the other warps scatter the block's own spikes along the rank's rows
//      into the increments of the step at which they act;
//   4. all warps scatter the received spikes;
//   5. grid-wide barrier (this GPU only).
//
// Increments live in a ring of `ring` rows per projection: a spike of step s from a
// population with synaptic delay d is added to row (s + 1 + d) % ring, and the update of
// step s consumes (and clears) row s % ring — the counterpart, for summed synaptic
// input, of the reference's delay ring buffer (brainstate/nn/_delay.py:768-958).  No
// spike list has to wait anywhere, whatever the delays.  When both delays are at least
// `slack` steps, a block consumes at step s the lists of step s - slack: the exchange
// latency then lies off the critical path (the lists have been in the inbox for
// `slack` steps when they are needed); the last `slack` lists are drained at the end of
// the launch so that nothing is pending between launches.
//
// With fixed_point the increments are 64-bit integers (weights scaled by 2^32 and
// rounded once): integer addition is associative, so the sums, and with them the spike
// raster, do not depend on the order of the atomic adds, the grid or the number of GPUs.
//
// Every wait is bounded.  A wait that runs out writes BSX_ERR_TIMEOUT into the status
// word; all blocks leave at the next step boundary.
#include "common.cuh"
#include "internal.cuh"
#include "network.cuh"

namespace bsx {

constexpr int kShThreads = 1024;
constexpr int kShWarps = kShThreads / 32;
constexpr int kShMaxPeers = 16;
constexpr int kShQueue = 2048;                 // received spikes a block stages for all its warps
constexpr int kShResMaxWords = 432;            // words per block with the state on chip (216 KB)
constexpr int kShMaxWords = 2048;              // words per block at all (own-spike offsets are 16 bit)

struct ShardDev {
  int64_t n_global, n_exc, first, n_local;
  ProjDev exc, inh;
  int chunk;
  float *V, *g_e, *g_i;
  int32_t* ref;
  void *incr_e, *incr_i;          // (ring, n_local) float or int64
  uint32_t* bits;                 // (ceil(n_local / 32)) local spike words of the last step, may be NULL
  int ring, delay_e, delay_i;
  bsx_lif_params_t p;
};

struct LinkDev {
  int world, rank, words_per_block, slots, slack;
  int64_t cap;                    // ids per list
  int64_t slot_stride;            // 64-bit words per inbox slot
  unsigned long long* inbox[kShMaxPeers];
  int32_t* sync;                  // [0] status word, [1] barrier counter
  int64_t spin_limit;
  int64_t seq0;
  int flags;                      // bit 0: push ids as soon as a warp has them; bit 1: fetch header and first ids together
};

// ---- increments: float (atomic order decides the last bit) or 2^-32 fixed point ----
template <bool FIXED>
struct Incr;
template <>
struct Incr<false> {
  using T = float;
  static __device__ __forceinline__ void add(T* p, float w) { red_add(p, w); }
  static __device__ __forceinline__ float value(T v) { return v; }
  static __device__ __forceinline__ bool nonzero(T v) { return v != 0.0f; }
};
template <>
struct Incr<true> {
  using T = long long;
  static __device__ __forceinline__ void add(T* p, float w) {
    const long long q = __float2ll_rn(__fmul_rn(w, 4294967296.0f));
    asm volatile("red.global.add.u64 [%0], %1;" ::"l"(p), "l"(q) : "memory");
  }
  static __device__ __forceinline__ float value(T v) { return __fmul_rn(__ll2float_rn(v), 2.3283064365386963e-10f); }
  static __device__ __forceinline__ bool nonzero(T v) { return v != 0; }
};

template <bool FIXED>
__device__ __forceinline__ void scatter_stub(const ProjDev& pr, int64_t row, int c, int chunk, int lane,
                                             typename Incr<FIXED>::T* __restrict__ out) {
  int64_t s, e;
  pr.rm.range(row, s, e);
  if (pr.cpr > 1) {   // fixed-number rows are cut into chunks; a CSR row is one item whatever its length
    s += (int64_t)c * chunk;
    if (s >= e) return;
    if (s + chunk < e) e = s + chunk;
  }
  if (!FIXED) {
    float* o = reinterpret_cast<float*>(out);
    if (pr.hetero) scatter_span<true>(pr.idx, pr.w, s, e, lane, 1.0f, o, pr.vec_ok);
    else scatter_span<false>(pr.idx, pr.w, s, e, lane, __ldg(pr.w), o, pr.vec_ok);
    return;
  }
  const float w0 = pr.hetero ? 0.0f : __ldg(pr.w);
#pragma unroll 4
  for (int64_t p = s + lane; p < e; p += 32)
    Incr<FIXED>::add(out + __ldg(pr.idx + p), pr.hetero ? __ldg(pr.w + p) : w0);
}

// One spike of global neuron `id`, fired at step `fired`: chunk c of its row goes to the
// increments of step fired + 1 + delay.
template <bool FIXED>
__device__ __forceinline__ void scatter_spike(const ShardDev& a, int64_t id, int c, int64_t fired, int lane) {
  using T = typename Incr<FIXED>::T;
  if (id < a.n_exc) {
    if (c < a.exc.cpr)
      scatter_stub<FIXED>(a.exc, id, c, a.chunk, lane,
                          reinterpret_cast<T*>(a.incr_e) + ((fired + 1 + a.delay_e) % a.ring) * a.n_local);
  } else {
    if (c < a.inh.cpr)
      scatter_stub<FIXED>(a.inh, id - a.n_exc, c, a.chunk, lane,
                          reinterpret_cast<T*>(a.incr_i) + ((fired + 1 + a.delay_i) % a.ring) * a.n_local);
  }
}

__device__ __forceinline__ void st_relaxed_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_relaxed_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Barrier over the blocks of this launch (all co-resident: cooperative launch).  The
// counter only grows; `target` is blocks * (barriers so far + 1).  Bounded: a block that
// waits too long records the timeout and goes on.  Returns the status word as thread 0 read
// it after the wait — the same value for every thread of the block, so the block can leave
// the step loop as one.
__device__ __forceinline__ int grid_barrier(int32_t* sync, unsigned target, int64_t spin_limit, int* s_status) {
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned* counter = reinterpret_cast<unsigned*>(sync + 1);
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(counter) : "memory");
    int64_t spins = 0;
    while (ld_acquire_gpu(counter) < target) {
      if (++spins > spin_limit) {
        atomicCAS(sync, 0, (int32_t)BSX_ERR_TIMEOUT);
        break;
      }
    }
    *s_status = *reinterpret_cast<volatile int32_t*>(sync);
  }
  __syncthreads();
  return *s_status;
}

// The block's own-spike list -> inbox of `peer`, list (source rank, source block) of slot seq % slots.
__device__ __forceinline__ void push_list(const LinkDev& L, int peer, int64_t seq, int count,
                                          const uint16_t* __restrict__ mine, int64_t gid0, int lane) {
  unsigned long long* base = L.inbox[peer] + (seq % L.slots) * L.slot_stride +
                             ((int64_t)L.rank * gridDim.x + blockIdx.x) * (1 + L.cap);
  const unsigned long long tag = (unsigned long long)(uint32_t)(seq + 1) << 32;
  if (!(L.flags & 1))                      // otherwise the ids went out while the update was running
    for (int k = lane; k < count; k += 32) st_relaxed_sys(base + 1 + k, tag | (uint32_t)(gid0 + mine[k]));
  if (lane == 0) st_relaxed_sys(base, tag | (uint32_t)count);
}

// Polls until the word carries `tag` (upper half); false when the patience runs out.
__device__ __forceinline__ bool wait_word(const unsigned long long* p, uint32_t tag, int64_t spin_limit,
                                          const int32_t* sync, uint32_t* payload) {
  int64_t spins = 0;
  for (;;) {
    const unsigned long long v = ld_relaxed_sys(p);
    if ((uint32_t)(v >> 32) == tag) {
      *payload = (uint32_t)v;
      return true;
    }
    if (++spins > spin_limit) return false;
    if ((spins & 1023) == 0 && *reinterpret_cast<const volatile int32_t*>(sync) != 0) return false;
  }
}

// One warp receives the list that block blockIdx.x of rank `src` pushed with sequence
// number `seq` (spikes fired at step `fired`): ids are staged in the block's queue for all
// warps; what does not fit is scattered by this warp right away.  Returns the count, or -1
// after a timeout.
template <bool FIXED>
__device__ __forceinline__ int recv_list(const ShardDev& a, const LinkDev& L, int src, int64_t seq, int64_t fired,
                                         int32_t* __restrict__ queue, int* __restrict__ queue_count, int cpr,
                                         int lane) {
  const unsigned long long* base = L.inbox[L.rank] + (seq % L.slots) * L.slot_stride +
                                   ((int64_t)src * gridDim.x + blockIdx.x) * (1 + L.cap);
  const uint32_t tag = (uint32_t)(seq + 1);
  uint32_t count = 0, id = 0;
  uint32_t k0 = 0;
  bool have_first = false;                // ids 0..30 already fetched by lanes 1..31
  if (L.flags & 2) {
    // header (lane 0) and the first 31 id words (lanes 1..31) in the same round trip: the
    // sender stores the ids before the header, so they are usually there with it
    int64_t spins = 0;
    unsigned long long v;
    for (;;) {
      v = ld_relaxed_sys(base + lane);
      const unsigned long long h = __shfl_sync(0xffffffffu, v, 0);
      if ((uint32_t)(h >> 32) == tag) {
        count = (uint32_t)h;
        break;
      }
      if (++spins > L.spin_limit) return -1;
      if ((spins & 1023) == 0 && *reinterpret_cast<const volatile int32_t*>(L.sync) != 0) return -1;
    }
    if ((int64_t)count > L.cap) return -1;
    int good = 1;
    if (lane >= 1 && (uint32_t)lane <= count) {
      if ((uint32_t)(v >> 32) == tag) id = (uint32_t)v;
      else good = wait_word(base + lane, tag, L.spin_limit, L.sync, &id) ? 1 : 0;
    }
    if (!__all_sync(0xffffffffu, good)) return -1;
    have_first = true;
  } else {
    int ok = 1;
    if (lane == 0) ok = wait_word(base, tag, L.spin_limit, L.sync, &count) ? 1 : 0;
    ok = __shfl_sync(0xffffffffu, ok, 0);
    count = __shfl_sync(0xffffffffu, count, 0);
    if (!ok || (int64_t)count > L.cap) return -1;
  }
  while (k0 < count) {
    int n;                                 // ids of this batch; lane `first + j` holds id k0 + j
    int first;
    if (have_first) {
      n = (int)(count < 31u ? count : 31u);
      first = 1;
      have_first = false;
    } else {
      const uint32_t k = k0 + lane;
      int good = 1;
      if (k < count) good = wait_word(base + 1 + k, tag, L.spin_limit, L.sync, &id) ? 1 : 0;
      if (!__all_sync(0xffffffffu, good)) return -1;
      n = (int)(count - k0 < 32u ? count - k0 : 32u);
      first = 0;
    }
    const int j0 = lane - first;           // position inside the batch
    int pos = 0;
    if (lane == 0) pos = atomicAdd(queue_count, n);
    pos = __shfl_sync(0xffffffffu, pos, 0);
    const bool in_batch = j0 >= 0 && j0 < n;
    const bool staged = in_batch && pos + j0 < kShQueue;
    if (staged) queue[pos + j0] = (int32_t)id;
    uint32_t direct = __ballot_sync(0xffffffffu, in_batch && !staged);
    while (direct) {
      const int j = __ffs(direct) - 1;
      direct &= direct - 1;
      const int64_t idj = (int64_t)__shfl_sync(0xffffffffu, id, j);
      for (int c = 0; c < cpr; ++c) scatter_spike<FIXED>(a, idj, c, fired, lane);
    }
    k0 += n;
  }
  return (int)count;
}

template <bool RESIDENT, bool FIXED, int MODEL = 0>
__global__ void __launch_bounds__(kShThreads, 1)
net_run_sharded_kernel(ShardDev a, LinkDev L, int steps, int64_t step0, uint32_t* __restrict__ raster,
                       int32_t* __restrict__ spike_counts) {
  using I = Incr<FIXED>;
  using T = typename I::T;
  constexpr int WPW = RESIDENT ? 8 : 4;                 // words a warp has in flight at once
  extern __shared__ __align__(16) unsigned char sh_raw[];
  __shared__ int s_spikes, s_queue_count, s_status;
  __shared__ int32_t s_queue[kShQueue];
  __shared__ unsigned long long* s_out[kShMaxPeers];      // this step's list in every peer's inbox
  const int cap = L.words_per_block * 32;
  float* sV = reinterpret_cast<float*>(sh_raw);
  float* sge = sV + (RESIDENT ? cap : 0);
  float* sgi = sge + (RESIDENT ? cap : 0);
  int16_t* sref = reinterpret_cast<int16_t*>(sgi + (RESIDENT ? cap : 0));
  uint16_t* smine = reinterpret_cast<uint16_t*>(sref + (RESIDENT ? cap : 0));   // own neurons that spiked this step
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  const int64_t words = (a.n_local + 31) >> 5;
  const int64_t word0 = (int64_t)blockIdx.x * L.words_per_block;
  int64_t my_words = words - word0;
  if (my_words > L.words_per_block) my_words = L.words_per_block;
  if (my_words < 0) my_words = 0;
  const int64_t n0 = word0 * 32;
  const int links = L.world - 1;                         // warps 0 .. links-1 talk to one peer each
  const int cpr = a.exc.cpr > a.inh.cpr ? a.exc.cpr : a.inh.cpr;
  if (RESIDENT) {
    for (int64_t li = tid; li < my_words * 32; li += kShThreads) {
      const int64_t i = n0 + li;
      const bool valid = i < a.n_local;
      sV[li] = valid ? a.V[i] : 0.0f;
      sge[li] = valid ? a.g_e[i] : 0.0f;
      sgi[li] = valid ? a.g_i[i] : 0.0f;
      sref[li] = valid ? (int16_t)a.ref[i] : (int16_t)0;
    }
  }
  __syncthreads();
  unsigned barriers = 0;
  int status = 0;
  for (int t = 0; t < steps; ++t) {
    const int64_t step = step0 + t;
    const int64_t seq = L.seq0 + t;
    T* __restrict__ cur_e = reinterpret_cast<T*>(a.incr_e) + (step % a.ring) * a.n_local;
    T* __restrict__ cur_i = reinterpret_cast<T*>(a.incr_i) + (step % a.ring) * a.n_local;
    if (tid == 0) {
      s_spikes = 0;
      s_queue_count = 0;
    }
    if (tid < links)
      s_out[tid] = L.inbox[(L.rank + 1 + tid) % L.world] + (seq % L.slots) * L.slot_stride +
                   ((int64_t)L.rank * gridDim.x + blockIdx.x) * (1 + L.cap);
    __syncthreads();
    const bool early = links > 0 && (L.flags & 1);
    const unsigned long long push_tag = (unsigned long long)(uint32_t)(seq + 1) << 32;
    // ---- 1. neuron update ----
    // (word and neuron numbers fit 32 bits: n_global < 2^31)
    const int my_w = (int)my_words, n0i = (int)n0, n_loc = (int)a.n_local;
    for (int wl0 = wid; wl0 < my_w; wl0 += kShWarps * WPW) {
      T de[WPW], di[WPW];
      float v[WPW], ge[WPW], gi[WPW];
      int32_t rr[WPW];
#pragma unroll
      for (int k = 0; k < WPW; ++k) {
        const int wl = wl0 + k * kShWarps;
        const int i = n0i + wl * 32 + lane;
        const bool valid = wl < my_w && i < n_loc;
        de[k] = valid ? cur_e[i] : T(0);
        di[k] = valid ? cur_i[i] : T(0);
        if (!RESIDENT) {
          v[k] = valid ? a.V[i] : 0.0f;
          ge[k] = valid ? a.g_e[i] : 0.0f;
          gi[k] = valid ? a.g_i[i] : 0.0f;
          rr[k] = valid ? a.ref[i] : 0;
        }
      }
#pragma unroll
      for (int k = 0; k < WPW; ++k) {
        const int wl = wl0 + k * kShWarps;
        if (wl >= my_w) break;                           // uniform across the warp
        const int li = wl * 32 + lane;
        const int i = n0i + li;
        bool spk = false;
        if (i < n_loc) {
          const int32_t r = RESIDENT ? (int32_t)sref[li] : rr[k];
          const NeuronOut o = neuron_math_m<MODEL>(a.p, I::value(de[k]), I::value(di[k]), RESIDENT ? sge[li] : ge[k],
                                          RESIDENT ? sgi[li] : gi[k], RESIDENT ? sV[li] : v[k], r,
                                          (uint32_t)a.first + (uint32_t)i, step);
          if (I::nonzero(de[k])) cur_e[i] = T(0);
          if (I::nonzero(di[k])) cur_i[i] = T(0);
          if (RESIDENT) {
            sge[li] = o.ge;
            sgi[li] = o.gi;
            sV[li] = o.V;
            if (o.r != r) sref[li] = (int16_t)o.r;
          } else {
            a.g_e[i] = o.ge;
            a.g_i[i] = o.gi;
            a.V[i] = o.V;
            if (o.r != r) a.ref[i] = o.r;
          }
          spk = o.spk;
          // NaN or infinity in the membrane potential or a synaptic variable (they propagate through the sum)
          if (!(fabsf(o.V) + fabsf(o.ge) + fabsf(o.gi) <= 3.0e38f)) atomicCAS(L.sync, 0, (int32_t)BSX_ERR_NONFINITE);
        }
        const uint32_t m = __ballot_sync(0xffffffffu, spk);
        if (lane == 0) {
          if (raster) raster[(int64_t)t * words + word0 + wl] = m;
          if (a.bits && t == steps - 1) a.bits[word0 + wl] = m;
        }
        if (m) {
          int base = 0;
          if (lane == 0) base = atomicAdd(&s_spikes, __popc(m));
          base = __shfl_sync(0xffffffffu, base, 0);
          if (spk) {
            const int pos = base + __popc(m & ((1u << lane) - 1u));
            smine[pos] = (uint16_t)li;
            if (early)       // the id is on its way to every peer before the rest of the block has finished
              for (int p = 0; p < links; ++p) st_relaxed_sys(s_out[p] + 1 + pos, push_tag | ((uint32_t)a.first + (uint32_t)i));
          }
        }
      }
    }
    __syncthreads();
    const int mine = s_spikes;
    // ---- 2./3. link warps push and receive; the others scatter the block's own spikes ----
    if (wid < links) {
      const int peer = (L.rank + 1 + wid) % L.world;
      push_list(L, peer, seq, mine, smine, a.first + n0, lane);
      if (t >= L.slack) {
        const int got = recv_list<FIXED>(a, L, peer, seq - L.slack, step - L.slack, s_queue, &s_queue_count, cpr, lane);
        if (lane == 0) {
          if (got < 0) atomicCAS(L.sync, 0, (int32_t)BSX_ERR_TIMEOUT);
          else if (got > 0 && spike_counts) atomicAdd(spike_counts + (t - L.slack), got);
        }
      }
    } else {
      const int items = mine * cpr;
      for (int it = wid - links; it < items; it += kShWarps - links) {
        const int q = it / cpr, c = it - q * cpr;
        scatter_spike<FIXED>(a, a.first + n0 + smine[q], c, step, lane);
      }
    }
    if (tid == 0 && mine && spike_counts) atomicAdd(spike_counts + t, mine);
    // ---- 4. received spikes, all warps ----
    if (links > 0) {
      __syncthreads();
      const int staged = s_queue_count < kShQueue ? s_queue_count : kShQueue;
      const int items = staged * cpr;
      for (int it = wid; it < items; it += kShWarps) {
        const int q = it / cpr, c = it - q * cpr;
        scatter_spike<FIXED>(a, s_queue[q], c, step - L.slack, lane);
      }
    }
    // ---- 5. every increment of the next step is in place once all blocks are here ----
    ++barriers;
    status = grid_barrier(L.sync, barriers * gridDim.x, L.spin_limit, &s_status);
    if (status != 0) break;                              // uniform across the block
  }
  // lists still in the inbox (the last `slack` steps): consume them before the launch ends
  if (links > 0 && L.slack > 0 && status == 0) {
    for (int t = steps - L.slack < 0 ? 0 : steps - L.slack; t < steps; ++t) {
      __syncthreads();
      if (tid == 0) s_queue_count = 0;
      __syncthreads();
      if (wid < links) {
        const int peer = (L.rank + 1 + wid) % L.world;
        const int got = recv_list<FIXED>(a, L, peer, L.seq0 + t, step0 + t, s_queue, &s_queue_count, cpr, lane);
        if (lane == 0) {
          if (got < 0) atomicCAS(L.sync, 0, (int32_t)BSX_ERR_TIMEOUT);
          else if (got > 0 && spike_counts) atomicAdd(spike_counts + t, got);
        }
      }
      __syncthreads();
      const int staged = s_queue_count < kShQueue ? s_queue_count : kShQueue;
      const int items = staged * cpr;
      for (int it = wid; it < items; it += kShWarps) {
        const int q = it / cpr, c = it - q * cpr;
        scatter_spike<FIXED>(a, s_queue[q], c, step0 + t, lane);
      }
    }
  }
  if (RESIDENT) {
    __syncthreads();
    for (int64_t li = tid; li < my_words * 32; li += kShThreads) {
      const int64_t i = n0 + li;
      if (i < a.n_local) {
        a.V[i] = sV[li];
        a.g_e[i] = sge[li];
        a.g_i[i] = sgi[li];
        a.ref[i] = sref[li];
      }
    }
  }
}

}  // namespace bsx

using namespace bsx;

extern "C" {

int bsx_net_shard_geometry(int64_t words_per_rank, int32_t* blocks, int32_t* words_per_block) {
  if (words_per_rank <= 0 || !blocks || !words_per_block) return fail(BSX_ERR_INVALID_ARG, "bad geometry request");
  const int sms = sm_count();
  if (sms <= 0) return fail(BSX_ERR_CUDA, "no CUDA device");
  int64_t wpb = (words_per_rank + sms - 1) / sms;
  if (wpb < kShWarps) wpb = kShWarps;                     // at least one word per warp
  if (wpb > kShMaxWords)
    return fail(BSX_ERR_UNSUPPORTED, "%lld spike words per rank exceed %d blocks of %d words",
                (long long)words_per_rank, sms, kShMaxWords);
  *words_per_block = (int32_t)wpb;
  *blocks = (int32_t)((words_per_rank + wpb - 1) / wpb);
  return BSX_OK;
}

size_t bsx_net_inbox_bytes(int32_t world, int32_t blocks, int32_t words_per_block, int32_t slots) {
  if (world < 1 || blocks < 1 || words_per_block < 1 || slots < 1) return 0;
  return (size_t)slots * (size_t)world * (size_t)blocks * (size_t)(1 + (int64_t)words_per_block * 32) * 8;
}

int bsx_net_run_sharded(const bsx_net_shard_t* net, const bsx_lif_params_t* params, const bsx_net_links_t* links,
                        int32_t steps, int64_t step0, uint32_t* raster, int32_t* spike_counts,
                        bsx_stream_t stream) {
  BSX_TRACE("bsx_net_run_sharded");
  if (!net || !params || !links) return fail(BSX_ERR_INVALID_ARG, "net, params or links is NULL");
  if (steps < 0 || step0 < 0 || links->seq0 < 0) return fail(BSX_ERR_INVALID_ARG, "bad step range");
  if (steps > (1 << 24)) return fail(BSX_ERR_UNSUPPORTED, "at most 2^24 steps per launch");
  if (net->n_global <= 0 || net->n_exc < 0 || net->n_exc > net->n_global || net->n_local < 0 || net->first < 0 ||
      net->first + net->n_local > net->n_global)
    return fail(BSX_ERR_INVALID_ARG, "inconsistent network sizes");
  if (net->n_global > INT32_MAX) return fail(BSX_ERR_UNSUPPORTED, "n_global must fit int32");
  if (net->first % 32) return fail(BSX_ERR_INVALID_ARG, "the first local neuron must be a multiple of 32");
  if (net->exc.n_pre != net->n_exc || net->inh.n_pre != net->n_global - net->n_exc ||
      net->exc.n_post != net->n_local || net->inh.n_post != net->n_local)
    return fail(BSX_ERR_INVALID_ARG,
                "projection shapes do not match the shard (rows: population, columns: local neurons)");
  if (net->n_local > 0 && (!net->V || !net->g_e || !net->g_i || !net->ref || !net->incr_e || !net->incr_i))
    return fail(BSX_ERR_INVALID_ARG, "a state buffer of the shard is NULL");
  if (net->delay_e < 0 || net->delay_i < 0) return fail(BSX_ERR_INVALID_ARG, "negative synaptic delay");
  const int dmax = net->delay_e > net->delay_i ? net->delay_e : net->delay_i;
  const int dmin = net->delay_e < net->delay_i ? net->delay_e : net->delay_i;
  if (net->ring < dmax + 2)
    return fail(BSX_ERR_INVALID_ARG, "the increment ring needs at least max(delay) + 2 = %d rows", dmax + 2);
  if (links->world < 1 || links->world > kShMaxPeers || links->rank < 0 || links->rank >= links->world)
    return fail(BSX_ERR_INVALID_ARG, "world must be 1..%d and rank inside it", kShMaxPeers);
  if (!links->sync) return fail(BSX_ERR_INVALID_ARG, "links->sync is NULL");
  if (links->blocks < 1 || links->words_per_block < kShWarps || links->words_per_block > kShMaxWords)
    return fail(BSX_ERR_INVALID_ARG, "blocks / words_per_block out of range (see bsx_net_shard_geometry)");
  if ((int64_t)links->blocks * links->words_per_block < (net->n_local + 31) / 32)
    return fail(BSX_ERR_INVALID_ARG, "blocks * words_per_block does not cover the shard");
  if (net->first != (int64_t)links->rank * links->words_per_rank * 32 && net->n_local > 0)
    return fail(BSX_ERR_INVALID_ARG, "first local neuron must be rank * words_per_rank * 32");
  if (links->slack < 0 || links->slack > dmin)
    return fail(BSX_ERR_INVALID_ARG, "slack must lie in [0, min(delay_e, delay_i)] = [0, %d]", dmin);
  if (links->world > 1) {
    if (links->slots < 2 * links->slack + 2)
      return fail(BSX_ERR_INVALID_ARG, "the inbox needs at least 2 * slack + 2 = %d slots", 2 * links->slack + 2);
    for (int r = 0; r < links->world; ++r)
      if (!links->inbox[r]) return fail(BSX_ERR_INVALID_ARG, "inbox of rank %d is NULL", r);
  }
  const int sms = sm_count();
  if (sms <= 0) return fail(BSX_ERR_CUDA, "no CUDA device");
  if (links->blocks > sms)
    return fail(BSX_ERR_UNSUPPORTED, "%d blocks cannot be resident together on %d SMs", links->blocks, sms);
  ShardDev a;
  a.chunk = 128;
  int64_t kmax = net->exc.conn_num > net->inh.conn_num ? net->exc.conn_num : net->inh.conn_num;
  while ((kmax + a.chunk - 1) / a.chunk > 64) a.chunk *= 2;
  int rc = make_proj(&net->exc, a.chunk, &a.exc);
  if (rc) return rc;
  rc = make_proj(&net->inh, a.chunk, &a.inh);
  if (rc) return rc;
  a.n_global = net->n_global;
  a.n_exc = net->n_exc;
  a.first = net->first;
  a.n_local = net->n_local;
  a.V = net->V; a.g_e = net->g_e; a.g_i = net->g_i; a.ref = net->ref;
  a.incr_e = net->incr_e; a.incr_i = net->incr_i;
  a.bits = net->bits;
  a.ring = net->ring;
  a.delay_e = net->delay_e;
  a.delay_i = net->delay_i;
  a.p = *params;
  LinkDev L;
  L.world = links->world;
  L.rank = links->rank;
  L.words_per_block = links->words_per_block;
  L.slots = links->slots > 0 ? links->slots : 2;
  L.slack = links->world > 1 ? links->slack : 0;
  L.cap = (int64_t)links->words_per_block * 32;
  L.slot_stride = (int64_t)links->world * links->blocks * (1 + L.cap);
  for (int r = 0; r < kShMaxPeers; ++r)
    L.inbox[r] = r < links->world ? reinterpret_cast<unsigned long long*>(links->inbox[r]) : nullptr;
  L.sync = links->sync;
  L.spin_limit = links->spin_limit > 0 ? links->spin_limit : (int64_t)1 << 21;
  L.seq0 = links->seq0;
  L.flags = links->flags;
  cudaStream_t st = as_stream(stream);
  if (spike_counts && steps > 0) BSX_CUDA(cudaMemsetAsync(spike_counts, 0, sizeof(int32_t) * (size_t)steps, st));
  if (steps == 0) return BSX_OK;
  BSX_CUDA(cudaMemsetAsync(links->sync + 1, 0, sizeof(int32_t), st));      // barrier counter of this launch
  const bool resident = links->words_per_block <= kShResMaxWords && params->ref_steps < 32768;
  const bool fixed = net->fixed_point != 0;
  const void* fn = resident ? (fixed ? (const void*)net_run_sharded_kernel<true, true>
                                     : (const void*)net_run_sharded_kernel<true, false>)
                            : (fixed ? (const void*)net_run_sharded_kernel<false, true>
                                     : (const void*)net_run_sharded_kernel<false, false>);
  // state in shared memory: the synapse model and the presence of a background drive are compile-time constants
  if (resident) {
    const int model = a.p.ext_threshold == 0 ? (a.p.coba ? 1 : 2) : (a.p.coba ? 0 : 3);
    if (model == 1) fn = fixed ? (const void*)net_run_sharded_kernel<true, true, 1> : (const void*)net_run_sharded_kernel<true, false, 1>;
    if (model == 2) fn = fixed ? (const void*)net_run_sharded_kernel<true, true, 2> : (const void*)net_run_sharded_kernel<true, false, 2>;
    if (model == 3) fn = fixed ? (const void*)net_run_sharded_kernel<true, true, 3> : (const void*)net_run_sharded_kernel<true, false, 3>;
  }
  const size_t per_neuron = (resident ? 3 * sizeof(float) + sizeof(int16_t) : 0) + sizeof(uint16_t);
  const size_t smem = (size_t)L.cap * per_neuron;
  BSX_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  int steps_i = steps;
  int64_t step0_i = step0;
  void* args[] = {&a, &L, &steps_i, &step0_i, &raster, &spike_counts};
  BSX_CUDA(cudaLaunchCooperativeKernel(fn, dim3((unsigned)links->blocks), dim3(kShThreads), args, smem, st));
  return BSX_OK;
}

}  // extern "C"
