// Fused E/I network step: event scatter -> exponential synapses -> LIF (current- or
// conductance-based) -> threshold / refractory -> packed spikes + spike list.
//
// This replaces, for one simulation step, the chain the reference's examples
// build from separate operators (examples/400_CUBA_2005_bpu.py:47-66:
// AlignPostProj(comm=EventFixedProb, syn=Expon, out=CUBA|COBA, post=LIFRef)):
//
//   phase A  for every neuron that spiked in the previous step, add its row of
//            weights into delta_e (excitatory rows) or delta_i (inhibitory rows);
//   phase B  g <- g*decay + delta (delta cleared in the same pass), membrane
//            update by the exponential-Euler rule of brainstate/nn/_exp_euler.py:226-249,
//            threshold, reset, refractory count, spike word by __ballot_sync and
//            append to the next spike list.
//
// Synaptic currents never leave the delta/g arrays: there is no current vector
// written to and re-read from HBM between the product and the neuron update.
// bsx_net_run keeps both phases of many steps in ONE cooperative launch
// (grid-wide barriers between phases); the split entry points serve the
// multi-GPU driver, which exchanges the spike words between phases.
//
// Every float operation below is a single IEEE operation (no fused multiply-add)
// and the exponential factor of the conductance-based rule is evaluated in double
// and rounded once, so spike rasters can be compared bit for bit with a CPU
// restatement that does the same.
#include <cooperative_groups.h>

#include "common.cuh"
#include "internal.cuh"
#include "network.cuh"

namespace cg = cooperative_groups;

namespace bsx {

struct NetDev {
  int64_t n_global, n_exc, first, n_local;
  ProjDev exc, inh;
  int chunk;
  float *V, *g_e, *g_i, *delta_e, *delta_i;
  int32_t* ref;
  uint32_t* bits;
  int32_t* lists;      // ring of spike lists, stride n_global + 1
  int ring, delay_e, delay_i;
  bsx_lif_params_t p;
  __device__ __forceinline__ int32_t* slot(int64_t step) const {
    return lists + (step % ring) * (n_global + 1);
  }
};

__device__ __forceinline__ void scatter_one(const ProjDev& pr, int64_t row, int c, int chunk, int lane,
                                            float* __restrict__ out) {
  int64_t s, e;
  pr.rm.range(row, s, e);
  if (pr.cpr > 1) {   // fixed-number rows are cut into chunks; a CSR row is one item whatever its length
    s += (int64_t)c * chunk;
    if (s >= e) return;
    if (s + chunk < e) e = s + chunk;
  }
  if (pr.hetero) scatter_span<true>(pr.idx, pr.w, s, e, lane, 1.0f, out, pr.vec_ok);
  else scatter_span<false>(pr.idx, pr.w, s, e, lane, __ldg(pr.w), out, pr.vec_ok);
}

// Phase A for one list = [count, global ids...]; do_exc / do_inh select which
// population's rows are taken from it (the two projections may have different delays).
__device__ __forceinline__ void scatter_list(const NetDev& a, const int32_t* __restrict__ list, bool do_exc,
                                             bool do_inh, int64_t warp, int64_t nwarps, int lane,
                                             int64_t from = 0, int64_t to = -1) {
  const int64_t count = list[0];
  if (to < 0 || to > count) to = count;
  const int cpr = a.exc.cpr > a.inh.cpr ? a.exc.cpr : a.inh.cpr;
  const int64_t items = to * cpr;
  for (int64_t it = from * cpr + warp; it < items; it += nwarps) {
    const int64_t q = it / cpr;
    const int c = (int)(it - q * cpr);
    const int64_t id = list[1 + q];
    if (id < a.n_exc) {
      if (do_exc && c < a.exc.cpr) scatter_one(a.exc, id, c, a.chunk, lane, a.delta_e);
    } else {
      if (do_inh && c < a.inh.cpr) scatter_one(a.inh, id - a.n_exc, c, a.chunk, lane, a.delta_i);
    }
  }
}

// Phase A of step `step`: excitatory spikes of step - 1 - delay_e, inhibitory spikes
// of step - 1 - delay_i (steps before 0 produced nothing).
__device__ __forceinline__ void phase_scatter(const NetDev& a, int64_t step, int64_t warp, int64_t nwarps,
                                              int lane) {
  const int64_t te = step - 1 - a.delay_e, ti = step - 1 - a.delay_i;
  if (te == ti) {
    if (te >= 0) scatter_list(a, a.slot(te), true, true, warp, nwarps, lane);
  } else {
    if (te >= 0) scatter_list(a, a.slot(te), true, false, warp, nwarps, lane);
    if (ti >= 0) scatter_list(a, a.slot(ti), false, true, warp, nwarps, lane);
  }
}

// Phase B is split in two so that a warp can have the loads of two words in flight
// before it computes either: one L2 round trip per pair instead of per word.
struct NeuronIn {
  float de, di, ge0, gi0, V;
  int32_t r;
  bool valid;
};

__device__ __forceinline__ NeuronIn load_neuron(const NetDev& a, int64_t i) {
  NeuronIn s;
  s.valid = i >= 0 && i < a.n_local;
  if (s.valid) {
    s.de = a.delta_e[i];
    s.di = a.delta_i[i];
    s.ge0 = a.g_e[i];
    s.gi0 = a.g_i[i];
    s.V = a.V[i];
    s.r = a.ref[i];
  }
  return s;
}

// Applies neuron_math to neuron i of the global-memory state; unchanged values are
// not rewritten.  Returns whether it spiked.
__device__ __forceinline__ bool step_neuron(const NetDev& a, int64_t i, int64_t step, const NeuronIn& s) {
  if (!s.valid) return false;
  const NeuronOut o = neuron_math(a.p, s.de, s.di, s.ge0, s.gi0, s.V, s.r, (uint32_t)(a.first + i), step);
  if (s.de != 0.0f) a.delta_e[i] = 0.0f;
  if (s.di != 0.0f) a.delta_i[i] = 0.0f;
  a.g_e[i] = o.ge;
  a.g_i[i] = o.gi;
  a.V[i] = o.V;
  if (o.r != s.r) a.ref[i] = o.r;
  return o.spk;
}

// Phase B for local words wd0 and wd1 (wd1 < 0: none); returns their spike words.
__device__ __forceinline__ void update_two_words(const NetDev& a, int64_t wd0, int64_t wd1, int lane,
                                                 int64_t step, uint32_t* m0, uint32_t* m1, bool* spk0,
                                                 bool* spk1) {
  const int64_t i0 = wd0 * 32 + lane, i1 = wd1 >= 0 ? wd1 * 32 + lane : -1;
  const NeuronIn s0 = load_neuron(a, i0);
  const NeuronIn s1 = load_neuron(a, i1);
  *spk0 = step_neuron(a, i0, step, s0);
  *spk1 = step_neuron(a, i1, step, s1);
  *m0 = __ballot_sync(0xffffffffu, *spk0);
  *m1 = __ballot_sync(0xffffffffu, *spk1);
}

__device__ __forceinline__ void append_spikes(uint32_t m, bool spk, int lane, int64_t gid, int32_t* __restrict__ list) {
  const int total = __popc(m);
  if (!total) return;
  int base = 0;
  if (lane == 0) base = atomicAdd(list, total);
  base = __shfl_sync(0xffffffffu, base, 0);
  if (spk) list[1 + base + __popc(m & ((1u << lane) - 1u))] = (int32_t)gid;
}

// ---- small networks: one thread block, state in shared memory ------------------------
// A few thousand neurons fit one SM: V, g_e, g_i, delta_e, delta_i and the refractory
// count live in shared memory for the whole run, the two phases of a step are
// separated by __syncthreads instead of grid-wide barriers, and the scatter uses
// shared-memory adds.  Same arithmetic, same spike lists and words in global memory.
// One SM updates about 2 000 neurons per microsecond, a grid-wide barrier costs about
// two: measured 3.5 us per step at 4 000 neurons against 4.1 for the cooperative
// kernel, 5.5 against 4.4 at 8 000 — hence the limit.
constexpr int kSmallMax = 4096;
constexpr int kSmallThreads = 1024;

__device__ __forceinline__ void smem_red(float* p, float v) {
  asm volatile("red.shared.add.f32 [%0], %1;" ::"r"((uint32_t)__cvta_generic_to_shared(p)), "f"(v) : "memory");
}

__device__ __forceinline__ void small_scatter_row(const ProjDev& pr, int64_t row, int lane, float* __restrict__ acc) {
  int64_t s, e;
  pr.rm.range(row, s, e);
  const float w0 = pr.hetero ? 1.0f : __ldg(pr.w);
  for (int64_t p = s + lane; p < e; p += 32)
    smem_red(acc + __ldg(pr.idx + p), pr.hetero ? __ldg(pr.w + p) : w0);
}

__device__ __forceinline__ void small_scatter_id(const NetDev& a, int64_t id, bool do_exc, bool do_inh, int lane,
                                                 float* __restrict__ sde, float* __restrict__ sdi) {
  if (id < a.n_exc) {
    if (do_exc) small_scatter_row(a.exc, id, lane, sde);
  } else if (do_inh) {
    small_scatter_row(a.inh, id - a.n_exc, lane, sdi);
  }
}

__global__ void __launch_bounds__(kSmallThreads, 1)
net_run_small_kernel(NetDev a, int steps, int64_t step0, uint32_t* __restrict__ raster,
                     int32_t* __restrict__ spike_counts) {
  extern __shared__ __align__(16) float sm_state[];
  const int n = (int)a.n_local;
  float* sV = sm_state;
  float* sge = sV + n;
  float* sgi = sge + n;
  float* sde = sgi + n;
  float* sdi = sde + n;
  int16_t* sref = reinterpret_cast<int16_t*>(sdi + n);
  // the spike lists of the last two steps also stay on chip (ids fit 16 bits here), so
  // that an undelayed projection never waits for global memory to learn who spiked
  uint16_t* slist0 = reinterpret_cast<uint16_t*>(sref + n);
  uint16_t* slist1 = slist0 + n;
  __shared__ int32_t s_count[2];
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  const int nwarps = kSmallThreads / 32;
  const int words = (n + 31) >> 5;
  for (int i = tid; i < n; i += kSmallThreads) {
    sV[i] = a.V[i]; sge[i] = a.g_e[i]; sgi[i] = a.g_i[i];
    sde[i] = a.delta_e[i]; sdi[i] = a.delta_i[i]; sref[i] = (int16_t)a.ref[i];
  }
  if (step0 > 0) {   // the list of the step before the first one, from global memory
    const int32_t* lp = a.slot(step0 - 1);
    const int cnt = lp[0];
    uint16_t* dst = ((step0 - 1) & 1) ? slist1 : slist0;
    for (int q = tid; q < cnt; q += kSmallThreads) dst[q] = (uint16_t)lp[1 + q];
    if (tid == 0) s_count[(step0 - 1) & 1] = cnt;
  } else if (tid == 0) {
    s_count[0] = s_count[1] = 0;
  }
  __syncthreads();
  for (int t = 0; t < steps; ++t) {
    const int64_t step = step0 + t;
    int32_t* lnext = a.slot(step);
    uint16_t* snext = (step & 1) ? slist1 : slist0;
    const uint16_t* sprev = (step & 1) ? slist0 : slist1;
    const int prev_cnt = s_count[(step & 1) ^ 1];
    __syncthreads();
    if (tid == 0) s_count[step & 1] = 0;
    // phase A: delayed spike lists -> shared-memory increments
    const int64_t te = step - 1 - a.delay_e, ti = step - 1 - a.delay_i;
    for (int pass = 0; pass < 2; ++pass) {
      const int64_t ts = pass == 0 ? te : ti;
      if (ts < 0 || (pass == 1 && ti == te)) continue;
      const bool do_exc = pass == 0, do_inh = pass == 1 || ti == te;
      if (ts == step - 1) {                       // previous step: on-chip list
        for (int q = wid; q < prev_cnt; q += nwarps) small_scatter_id(a, sprev[q], do_exc, do_inh, lane, sde, sdi);
      } else {                                    // older step: its list in global memory
        const int32_t* lp = a.slot(ts);
        const int cnt = lp[0];
        for (int q = wid; q < cnt; q += nwarps) small_scatter_id(a, lp[1 + q], do_exc, do_inh, lane, sde, sdi);
      }
    }
    __syncthreads();
    // phase B
    for (int wd = wid; wd < words; wd += nwarps) {
      const int i = wd * 32 + lane;
      bool spk = false;
      if (i < n) {
        const NeuronOut o = neuron_math(a.p, sde[i], sdi[i], sge[i], sgi[i], sV[i], sref[i], (uint32_t)i, step);
        sde[i] = 0.0f; sdi[i] = 0.0f;
        sge[i] = o.ge; sgi[i] = o.gi; sV[i] = o.V; sref[i] = (int16_t)o.r;
        spk = o.spk;
      }
      const uint32_t m = __ballot_sync(0xffffffffu, spk);
      if (lane == 0) {
        a.bits[wd] = m;
        if (raster) raster[(int64_t)t * words + wd] = m;
      }
      const int total = __popc(m);
      if (total) {
        int base = 0;
        if (lane == 0) base = atomicAdd(&s_count[step & 1], total);
        base = __shfl_sync(0xffffffffu, base, 0);
        if (spk) {
          const int pos = base + __popc(m & ((1u << lane) - 1u));
          snext[pos] = (uint16_t)i;
          lnext[1 + pos] = i;               // the copy that outlives the launch (and serves delays)
        }
      }
    }
    __syncthreads();
    if (tid == 0) {
      const int c = s_count[step & 1];
      lnext[0] = c;
      if (spike_counts) spike_counts[t] = c;
    }
  }
  __syncthreads();
  for (int i = tid; i < n; i += kSmallThreads) {
    a.V[i] = sV[i]; a.g_e[i] = sge[i]; a.g_i[i] = sgi[i];
    a.delta_e[i] = sde[i]; a.delta_i[i] = sdi[i]; a.ref[i] = sref[i];
  }
}

// ---- one cooperative launch for many steps (single GPU) ------------------------
constexpr int kRunWords = 4;
__global__ void __launch_bounds__(256)
net_run_kernel(NetDev a, int steps, int64_t step0, uint32_t* __restrict__ raster,
               int32_t* __restrict__ spike_counts) {
  cg::grid_group grid = cg::this_grid();
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int64_t words = (a.n_local + 31) >> 5;
  for (int t = 0; t < steps; ++t) {
    const int64_t step = step0 + t;
    int32_t* lnext = a.slot(step);   // not among the slots read this step: ring >= max delay + 2
    if (warp == 0 && lane == 0) lnext[0] = 0;
    phase_scatter(a, step, warp, nwarps, lane);
    grid.sync();
    // four words per warp and round trip: networks too large for the resident kernel are bound
    // by the latency of the state loads, not by their bandwidth
    for (int64_t wd0 = warp; wd0 < words; wd0 += kRunWords * nwarps) {
      NeuronIn in[kRunWords];
#pragma unroll
      for (int k = 0; k < kRunWords; ++k) {
        const int64_t wd = wd0 + k * nwarps;
        in[k] = load_neuron(a, wd < words ? wd * 32 + lane : -1);
      }
#pragma unroll
      for (int k = 0; k < kRunWords; ++k) {
        const int64_t wd = wd0 + k * nwarps;
        if (wd >= words) break;                          // uniform across the warp
        const bool spk = step_neuron(a, wd * 32 + lane, step, in[k]);
        const uint32_t m = __ballot_sync(0xffffffffu, spk);
        if (lane == 0) {
          a.bits[wd] = m;
          if (raster) raster[(int64_t)t * words + wd] = m;
        }
        append_spikes(m, spk, lane, wd * 32 + lane, lnext);
      }
    }
    grid.sync();
    if (spike_counts && warp == 0 && lane == 0) spike_counts[t] = lnext[0];
  }
}

// ---- the same, with the neuron state resident in shared memory --------------------
// 148 SMs hold 33 MB of shared memory: up to about two million neurons can keep V, g_e,
// g_i (float32) and the refractory count (int16) on chip for the whole run, one 1024-thread
// block per SM owning a contiguous range of spike words.  Per step a neuron then costs one
// read of its two synaptic increments from L2 (and a store where they were not zero)
// instead of a read and a write of its whole state; all increments of a warp's words are
// requested before the first is used.  The increments stay in global memory because
// every SM scatters into them.  Arithmetic, spike words, lists and raster are those of
// net_run_kernel; the state is read from global memory at the start and written back at
// the end of the launch.
//
// ONE_BARRIER (projections without delay): a block scatters the spikes of its own neurons
// right after it has updated them, so nothing waits for the complete spike list and a step
// needs one grid-wide barrier instead of two.  A fast block must not add step t+1's
// increments to a neuron whose owner has not consumed step t's yet, so the increments are
// double-buffered by step parity; the second pair of buffers are the V and g_e arrays in
// global memory, which nobody reads while the state is on chip (they are cleared at the
// start and rewritten with the state at the end).  The spikes of the step before the launch
// come from their list, as in every other kernel, and the last step of a launch leaves its
// spikes to the list, so launches can be chained and mixed with the other kernels.
constexpr int kResThreads = 1024;
constexpr int kResWarps = kResThreads / 32;
constexpr int kResWordsPerWarp = 8;                       // words a warp has in flight at once
constexpr int kResMaxWords = 432;                         // words (of 32 neurons) per block: 216 KB
constexpr int kResBytesPerNeuron = 3 * sizeof(float) + 2 * sizeof(int16_t);   // state + own-spike list

template <bool ONE_BARRIER>
__global__ void __launch_bounds__(kResThreads, 1)
net_run_resident_kernel(NetDev a, int steps, int64_t step0, uint32_t* __restrict__ raster,
                        int32_t* __restrict__ spike_counts, int words_per_block) {
  cg::grid_group grid = cg::this_grid();
  extern __shared__ __align__(16) unsigned char res_raw[];
  __shared__ int s_spikes;
  const int cap = words_per_block * 32;
  float* sV = reinterpret_cast<float*>(res_raw);
  float* sge = sV + cap;
  float* sgi = sge + cap;
  int16_t* sref = reinterpret_cast<int16_t*>(sgi + cap);
  uint16_t* smine = reinterpret_cast<uint16_t*>(sref + cap);      // neurons of this block that spiked this step
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int64_t words = (a.n_local + 31) >> 5;
  const int64_t word0 = (int64_t)blockIdx.x * words_per_block;
  int64_t my_words = words - word0;
  if (my_words > words_per_block) my_words = words_per_block;
  if (my_words < 0) my_words = 0;
  const int64_t n0 = word0 * 32;
  for (int64_t li = tid; li < my_words * 32; li += kResThreads) {
    const int64_t i = n0 + li;
    const bool valid = i < a.n_local;
    sV[li] = valid ? a.V[i] : 0.0f;
    sge[li] = valid ? a.g_e[i] : 0.0f;
    sgi[li] = valid ? a.g_i[i] : 0.0f;
    sref[li] = valid ? (int16_t)a.ref[i] : (int16_t)0;
  }
  __syncthreads();
  if (ONE_BARRIER) {
    // every block reads only its own part of V and g_e, so they can be cleared right away
    for (int64_t li = tid; li < my_words * 32; li += kResThreads) {
      const int64_t i = n0 + li;
      if (i < a.n_local) {
        a.V[i] = 0.0f;
        a.g_e[i] = 0.0f;
      }
    }
    if (warp == 0 && lane == 0) a.slot(step0)[0] = 0;
    phase_scatter(a, step0, warp, nwarps, lane);          // the spikes of step0 - 1, from their list
    grid.sync();
  }
  const int cpr = a.exc.cpr > a.inh.cpr ? a.exc.cpr : a.inh.cpr;
  for (int t = 0; t < steps; ++t) {
    const int64_t step = step0 + t;
    int32_t* lnext = a.slot(step);   // not among the slots read this step: ring >= max delay + 2
    if (!ONE_BARRIER) {
      if (warp == 0 && lane == 0) lnext[0] = 0;
      phase_scatter(a, step, warp, nwarps, lane);
      grid.sync();
    }
    const bool odd = ONE_BARRIER && (t & 1);
    float* __restrict__ de_cur = odd ? a.V : a.delta_e;
    float* __restrict__ di_cur = odd ? a.g_e : a.delta_i;
    float* __restrict__ de_nxt = odd ? a.delta_e : a.V;
    float* __restrict__ di_nxt = odd ? a.delta_i : a.g_e;
    const bool pass_on = ONE_BARRIER && t + 1 < steps;     // the last step leaves its spikes to the list
    if (ONE_BARRIER) {
      if (tid == 0) s_spikes = 0;
      if (pass_on && warp == 0 && lane == 0) a.slot(step + 1)[0] = 0;   // no list is read in this mode
      __syncthreads();
    }
    for (int64_t wl0 = wid; wl0 < my_words; wl0 += kResWarps * kResWordsPerWarp) {
      float de[kResWordsPerWarp], di[kResWordsPerWarp];
#pragma unroll
      for (int k = 0; k < kResWordsPerWarp; ++k) {
        const int64_t wl = wl0 + (int64_t)k * kResWarps;
        const int64_t i = n0 + wl * 32 + lane;
        const bool valid = wl < my_words && i < a.n_local;
        de[k] = valid ? de_cur[i] : 0.0f;
        di[k] = valid ? di_cur[i] : 0.0f;
      }
#pragma unroll
      for (int k = 0; k < kResWordsPerWarp; ++k) {
        const int64_t wl = wl0 + (int64_t)k * kResWarps;
        if (wl >= my_words) break;                       // uniform across the warp
        const int64_t li = wl * 32 + lane;
        const int64_t i = n0 + li;
        bool spk = false;
        if (i < a.n_local) {
          const int32_t r = sref[li];
          const NeuronOut o = neuron_math(a.p, de[k], di[k], sge[li], sgi[li], sV[li], r, (uint32_t)(a.first + i), step);
          if (de[k] != 0.0f) de_cur[i] = 0.0f;
          if (di[k] != 0.0f) di_cur[i] = 0.0f;
          sge[li] = o.ge;
          sgi[li] = o.gi;
          sV[li] = o.V;
          if (o.r != r) sref[li] = (int16_t)o.r;
          spk = o.spk;
        }
        const uint32_t m = __ballot_sync(0xffffffffu, spk);
        const int64_t wd = word0 + wl;
        if (lane == 0) {
          a.bits[wd] = m;
          if (raster) raster[(int64_t)t * words + wd] = m;
        }
        append_spikes(m, spk, lane, i, lnext);
        if (pass_on && m) {
          int base = 0;
          if (lane == 0) base = atomicAdd(&s_spikes, __popc(m));
          base = __shfl_sync(0xffffffffu, base, 0);
          if (spk) smine[base + __popc(m & ((1u << lane) - 1u))] = (uint16_t)li;
        }
      }
    }
    if (pass_on) {
      __syncthreads();
      const int items = s_spikes * cpr;
      for (int it = wid; it < items; it += kResWarps) {
        const int q = it / cpr, c = it - q * cpr;
        const int64_t id = a.first + n0 + smine[q];
        if (id < a.n_exc) {
          if (c < a.exc.cpr) scatter_one(a.exc, id, c, a.chunk, lane, de_nxt);
        } else {
          if (c < a.inh.cpr) scatter_one(a.inh, id - a.n_exc, c, a.chunk, lane, di_nxt);
        }
      }
    }
    grid.sync();
    if (spike_counts && warp == 0 && lane == 0) spike_counts[t] = lnext[0];
  }
  for (int64_t li = tid; li < my_words * 32; li += kResThreads) {
    const int64_t i = n0 + li;
    if (i < a.n_local) {
      a.V[i] = sV[li];
      a.g_e[i] = sge[li];
      a.g_i[i] = sgi[li];
      a.ref[i] = sref[li];
    }
  }
}

// ---- split phases (multi-GPU driver) ----------------------------------------------
__global__ void __launch_bounds__(256) net_scatter_kernel(NetDev a, int64_t step) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  phase_scatter(a, step, warp, nwarps, lane);
}

// Phase A restricted to one section of every list: entries [0, mark) (`rest` == 0) or
// [mark, count) (`rest` != 0), where marks[slot] is the list's length when its first section
// was complete.  A driver that lists its own spikes first can scatter them while the other
// ranks' spike words are still on their way.
__global__ void __launch_bounds__(256)
net_scatter_part_kernel(NetDev a, int64_t step, const int32_t* __restrict__ marks, int rest) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int64_t te = step - 1 - a.delay_e, ti = step - 1 - a.delay_i;
  if (te >= 0) {
    const int64_t mk = marks[te % a.ring];
    scatter_list(a, a.slot(te), true, te == ti, warp, nwarps, lane, rest ? mk : 0, rest ? -1 : mk);
  }
  if (ti >= 0 && ti != te) {
    const int64_t mk = marks[ti % a.ring];
    scatter_list(a, a.slot(ti), false, true, warp, nwarps, lane, rest ? mk : 0, rest ? -1 : mk);
  }
}

__global__ void __launch_bounds__(256)
net_update_kernel(NetDev a, int64_t step, int32_t* __restrict__ local_count) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int64_t words = (a.n_local + 31) >> 5;
  const int64_t word0 = a.first >> 5;
  int mine = 0;
  for (int64_t wd = warp; wd < words; wd += 2 * nwarps) {
    const int64_t wd1 = wd + nwarps < words ? wd + nwarps : -1;
    bool spk0, spk1;
    uint32_t m0, m1;
    update_two_words(a, wd, wd1, lane, step, &m0, &m1, &spk0, &spk1);
    if (lane == 0) {
      a.bits[word0 + wd] = m0;
      if (wd1 >= 0) a.bits[word0 + wd1] = m1;
    }
    mine += __popc(m0) + __popc(m1);
  }
  if (local_count && lane == 0 && mine) atomicAdd(local_count, mine);
}


// Compacts the packed spike words of the whole network into a list of global ids.
__global__ void __launch_bounds__(256)
net_list_kernel(const uint32_t* __restrict__ bits, int64_t n_global, int32_t* __restrict__ list,
                int64_t word0 = 0, int64_t word1 = -1, int64_t skip0 = 0, int64_t skip1 = 0) {
  const int lane = threadIdx.x & 31;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  const int64_t all_words = (n_global + 31) >> 5;
  const int64_t words = word1 < 0 || word1 > all_words ? all_words : word1;
  for (int64_t g0 = word0 + tid - lane; g0 < words; g0 += nthreads) {
    const int64_t g = g0 + lane;
    uint32_t m = 0;
    if (g < words && !(g >= skip0 && g < skip1)) {
      m = bits[g];
      const int64_t left = n_global - g * 32;
      if (left < 32) m &= (1u << left) - 1u;
    }
    // warp-aggregated reservation of popc(m) slots per lane
    uint32_t cnt = __popc(m), incl = cnt;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    const uint32_t total = __shfl_sync(0xffffffffu, incl, 31);
    uint32_t base = 0;
    if (lane == 31 && total) base = (uint32_t)atomicAdd(list, (int32_t)total);
    base = __shfl_sync(0xffffffffu, base, 31);
    uint32_t pos = base + incl - cnt;
    while (m) {
      const int k = __ffs(m) - 1;
      m &= m - 1;
      list[1 + pos++] = (int32_t)(g * 32 + k);
    }
  }
}

static int make_net(const bsx_net_t* net, const bsx_lif_params_t* p, NetDev* a) {
  if (!net) return fail(BSX_ERR_INVALID_ARG, "net is NULL");
  if (net->n_global <= 0 || net->n_exc < 0 || net->n_exc > net->n_global || net->n_local < 0 ||
      net->first < 0 || net->first + net->n_local > net->n_global)
    return fail(BSX_ERR_INVALID_ARG, "inconsistent network sizes");
  if (net->n_global > INT32_MAX) return fail(BSX_ERR_UNSUPPORTED, "n_global must fit int32");
  if (net->first % 32) return fail(BSX_ERR_INVALID_ARG, "the first local neuron must be a multiple of 32");
  if (net->exc.n_pre != net->n_exc || net->inh.n_pre != net->n_global - net->n_exc ||
      net->exc.n_post != net->n_local || net->inh.n_post != net->n_local)
    return fail(BSX_ERR_INVALID_ARG, "projection shapes do not match the network (rows: population, columns: local neurons)");
  if (!net->V || !net->g_e || !net->g_i || !net->ref || !net->delta_e || !net->delta_i || !net->bits ||
      !net->lists)
    return fail(BSX_ERR_INVALID_ARG, "a state buffer of the network is NULL");
  if (net->delay_e < 0 || net->delay_i < 0) return fail(BSX_ERR_INVALID_ARG, "negative synaptic delay");
  {
    const int dmax = net->delay_e > net->delay_i ? net->delay_e : net->delay_i;
    if (net->ring < dmax + 2)
      return fail(BSX_ERR_INVALID_ARG, "the spike-list ring needs at least max(delay) + 2 = %d lists", dmax + 2);
  }
  a->chunk = 128;
  // keep chunks-per-row small for very long rows
  int64_t kmax = net->exc.conn_num > net->inh.conn_num ? net->exc.conn_num : net->inh.conn_num;
  while ((kmax + a->chunk - 1) / a->chunk > 64) a->chunk *= 2;
  int rc = make_proj(&net->exc, a->chunk, &a->exc);
  if (rc) return rc;
  rc = make_proj(&net->inh, a->chunk, &a->inh);
  if (rc) return rc;
  a->n_global = net->n_global;
  a->n_exc = net->n_exc;
  a->first = net->first;
  a->n_local = net->n_local;
  a->V = net->V; a->g_e = net->g_e; a->g_i = net->g_i; a->ref = net->ref;
  a->delta_e = net->delta_e; a->delta_i = net->delta_i;
  a->bits = net->bits;
  a->lists = net->lists;
  a->ring = net->ring;
  a->delay_e = net->delay_e;
  a->delay_i = net->delay_i;
  if (p) a->p = *p; else a->p = bsx_lif_params_t{};
  return BSX_OK;
}

}  // namespace bsx

using namespace bsx;

extern "C" {

int bsx_net_run(const bsx_net_t* net, const bsx_lif_params_t* params, int32_t steps, int64_t step0,
                uint32_t* raster, int32_t* spike_counts, int32_t blocks, bsx_stream_t stream) {
  BSX_TRACE("bsx_net_run");
  if (!params) return fail(BSX_ERR_INVALID_ARG, "params is NULL");
  if (steps < 0 || step0 < 0) return fail(BSX_ERR_INVALID_ARG, "bad step range");
  NetDev a;
  int rc = make_net(net, params, &a);
  if (rc) return rc;
  if (net->first != 0 || net->n_local != net->n_global)
    return fail(BSX_ERR_INVALID_ARG, "bsx_net_run drives a whole network on one GPU (first = 0, n_local = n_global)");
  if (steps == 0) return BSX_OK;
  int sms = sm_count();
  if (sms <= 0) return fail(BSX_ERR_CUDA, "no CUDA device");
  // the whole network fits one SM's shared memory (refractory counts are kept as int16 there)
  if (blocks == 0 && net->n_global <= kSmallMax && params->ref_steps < 32768) {
    const size_t smem = (size_t)net->n_global * (5 * sizeof(float) + 3 * sizeof(int16_t));
    BSX_CUDA(cudaFuncSetAttribute(net_run_small_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    net_run_small_kernel<<<1, kSmallThreads, smem, as_stream(stream)>>>(a, steps, step0, raster, spike_counts);
    BSX_LAUNCH_CHECK("net_run_small_kernel");
    return BSX_OK;
  }
  int steps_i = steps;
  int64_t step0_i = step0;
  // the neuron state fits the shared memory of the SMs: one resident block per SM
  const int64_t words = (net->n_local + 31) / 32;
  if (blocks == 0 && params->ref_steps < 32768 && words <= (int64_t)sms * kResMaxWords) {
    int64_t wpb = (words + sms - 1) / sms;
    if (wpb < kResWarps) wpb = kResWarps;                  // at least one word per warp
    const int64_t grid_blocks = (words + wpb - 1) / wpb;
    int wpb_i = (int)wpb;
    const size_t smem = (size_t)wpb * 32 * kResBytesPerNeuron;
    const bool one_barrier = a.delay_e == 0 && a.delay_i == 0;
    const void* fn = one_barrier ? (const void*)net_run_resident_kernel<true> : (const void*)net_run_resident_kernel<false>;
    BSX_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    void* rargs[] = {&a, &steps_i, &step0_i, &raster, &spike_counts, &wpb_i};
    BSX_CUDA(cudaLaunchCooperativeKernel(fn, dim3((unsigned)grid_blocks), dim3(kResThreads), rargs, smem,
                                         as_stream(stream)));
    return BSX_OK;
  }
  int per_sm = 0;
  BSX_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, net_run_kernel, 256, 0));
  if (per_sm < 1) return fail(BSX_ERR_CUDA, "the network kernel does not fit on an SM");
  int64_t max_blocks = (int64_t)sms * (per_sm < 4 ? per_sm : 4);
  int64_t want = blocks > 0 ? blocks : (net->n_local + 255) / 256;
  if (want < 1) want = 1;
  if (want > max_blocks) want = max_blocks;
  void* args[] = {&a, &steps_i, &step0_i, &raster, &spike_counts};
  BSX_CUDA(cudaLaunchCooperativeKernel((const void*)net_run_kernel, dim3((unsigned)want), dim3(256), args, 0,
                                       as_stream(stream)));
  return BSX_OK;
}

int bsx_net_scatter(const bsx_net_t* net, int64_t step, bsx_stream_t stream) {
  BSX_TRACE("bsx_net_scatter");
  if (step < 0) return fail(BSX_ERR_INVALID_ARG, "negative step");
  NetDev a;
  int rc = make_net(net, nullptr, &a);
  if (rc) return rc;
  int sms = sm_count();
  if (sms <= 0) return fail(BSX_ERR_CUDA, "no CUDA device");
  net_scatter_kernel<<<(unsigned)(sms * 4), 256, 0, as_stream(stream)>>>(a, step);
  BSX_LAUNCH_CHECK("net_scatter_kernel");
  return BSX_OK;
}

int bsx_net_update(const bsx_net_t* net, const bsx_lif_params_t* params, int64_t step, int32_t* local_count,
                   bsx_stream_t stream) {
  BSX_TRACE("bsx_net_update");
  if (!params) return fail(BSX_ERR_INVALID_ARG, "params is NULL");
  if (step < 0) return fail(BSX_ERR_INVALID_ARG, "negative step");
  NetDev a;
  int rc = make_net(net, params, &a);
  if (rc) return rc;
  if (net->n_local == 0) return BSX_OK;
  int sms = sm_count();
  if (sms <= 0) return fail(BSX_ERR_CUDA, "no CUDA device");
  int64_t blocks = (net->n_local + 255) / 256;
  if (blocks > (int64_t)sms * 8) blocks = (int64_t)sms * 8;
  net_update_kernel<<<(unsigned)blocks, 256, 0, as_stream(stream)>>>(a, step, local_count);
  BSX_LAUNCH_CHECK("net_update_kernel");
  return BSX_OK;
}

int bsx_net_list_from_bits(const bsx_net_t* net, int64_t step, bsx_stream_t stream) {
  BSX_TRACE("bsx_net_list_from_bits");
  if (step < 0) return fail(BSX_ERR_INVALID_ARG, "negative step");
  NetDev a;
  int rc = make_net(net, nullptr, &a);
  if (rc) return rc;
  int sms = sm_count();
  if (sms <= 0) return fail(BSX_ERR_CUDA, "no CUDA device");
  int32_t* list = net->lists + (step % net->ring) * (net->n_global + 1);
  BSX_CUDA(cudaMemsetAsync(list, 0, sizeof(int32_t), as_stream(stream)));
  const int64_t words = (a.n_global + 31) >> 5;
  int64_t blocks = (words + 255) / 256;
  if (blocks > (int64_t)sms * 4) blocks = (int64_t)sms * 4;
  if (blocks < 1) blocks = 1;
  net_list_kernel<<<(unsigned)blocks, 256, 0, as_stream(stream)>>>(a.bits, a.n_global, list);
  BSX_LAUNCH_CHECK("net_list_kernel");
  return BSX_OK;
}

int bsx_net_scatter_part(const bsx_net_t* net, int64_t step, const int32_t* marks, int32_t rest, bsx_stream_t stream) {
  BSX_TRACE("bsx_net_scatter_part");
  if (step < 0) return fail(BSX_ERR_INVALID_ARG, "negative step");
  if (!marks) return fail(BSX_ERR_INVALID_ARG, "marks is NULL");
  NetDev a;
  int rc = make_net(net, nullptr, &a);
  if (rc) return rc;
  int sms = sm_count();
  if (sms <= 0) return fail(BSX_ERR_CUDA, "no CUDA device");
  net_scatter_part_kernel<<<(unsigned)(sms * 4), 256, 0, as_stream(stream)>>>(a, step, marks, rest);
  BSX_LAUNCH_CHECK("net_scatter_part_kernel");
  return BSX_OK;
}

int bsx_net_list_from_bits_part(const bsx_net_t* net, int64_t step, int64_t word0, int64_t word1, int32_t rest,
                                int32_t* marks, bsx_stream_t stream) {
  BSX_TRACE("bsx_net_list_from_bits_part");
  if (step < 0) return fail(BSX_ERR_INVALID_ARG, "negative step");
  NetDev a;
  int rc = make_net(net, nullptr, &a);
  if (rc) return rc;
  const int64_t words = (a.n_global + 31) >> 5;
  if (word0 < 0 || word1 < word0 || word1 > words) return fail(BSX_ERR_INVALID_ARG, "word range outside the network");
  if (!rest && !marks) return fail(BSX_ERR_INVALID_ARG, "marks is NULL");
  int sms = sm_count();
  if (sms <= 0) return fail(BSX_ERR_CUDA, "no CUDA device");
  cudaStream_t st = as_stream(stream);
  int32_t* list = net->lists + (step % net->ring) * (net->n_global + 1);
  const int64_t span = rest ? words : word1 - word0;
  int64_t blocks = (span + 255) / 256;
  if (blocks > (int64_t)sms * 4) blocks = (int64_t)sms * 4;
  if (blocks < 1) blocks = 1;
  if (!rest) {
    // first section: the words [word0, word1) into an emptied list; its length becomes the mark
    BSX_CUDA(cudaMemsetAsync(list, 0, sizeof(int32_t), st));
    net_list_kernel<<<(unsigned)blocks, 256, 0, st>>>(a.bits, a.n_global, list, word0, word1, 0, 0);
    BSX_LAUNCH_CHECK("net_list_kernel");
    BSX_CUDA(cudaMemcpyAsync(marks + (step % net->ring), list, sizeof(int32_t), cudaMemcpyDeviceToDevice, st));
  } else {
    // second section: every other word, appended
    net_list_kernel<<<(unsigned)blocks, 256, 0, st>>>(a.bits, a.n_global, list, 0, -1, word0, word1);
    BSX_LAUNCH_CHECK("net_list_kernel");
  }
  return BSX_OK;
}

// Host restatement of the device hash, for bindings that want to predict the drive.
uint32_t bsx_drive_hash(uint32_t seed, uint32_t neuron, uint32_t step) { return drive_hash(seed, neuron, step); }

}  // extern "C"
