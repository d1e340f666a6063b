// Batched pre-centric scatter with the output held in shared memory.
//
// For a batch of spike vectors and a modest number of postsynaptic neurons, one
// thread block owns a slice of up to 32 768 columns of ONE batch row's output and keeps
// it in shared memory (128 KB).  The block lists the active presynaptic rows of its
// spike vector (count, block-wide scan, write: one round when they fit the 2048-entry
// list, rounds over spans sized to the density otherwise) and fetches all their ranges at once, then its warps take rows from the list
// one at a time, issue all 128-bit index and weight loads of a 384-entry stretch before
// touching any of them, and add the entries that fall into the slice with shared-memory
// atomics — about four times the rate of red.global.add.f32.  The slice is written to
// global memory once, coalesced: no workspace, no separate clearing of the output.
// With n_post = 65 536 two blocks share a batch row.  Over the original rows each of them reads
// every active row (the two are neighbours in launch order, so the second read is served by
// L2); over the sliced copy (rows regrouped by slice, bsx_sliced_build) each reads only its own
// groups, the blocks of one slice are launched together, and every warp prefetches into L2 the
// group that is handed out one round later.  The compressed form of the sliced copy stores
// 16-bit column offsets inside the slice and the weights in fixed point.  Beyond four slices
// the re-reading outweighs any gain.  Like every atomic scatter, the
// summation order of heterogeneous weights is not fixed.  With homogeneous weights and
// an event input every event adds the same value, so the slice holds integer hit counts
// (native integer atomics, no compare-and-swap loop) and every output is count * weight,
// rounded once: exact in the count, and within an ulp of — not bit-equal to — a sequential
// float sum of `count` copies of the weight.
//
// One block per SM: the kernel needs batch * slices >= the number of SMs to fill the
// GPU, which is what the automatic choice in vecmat_common checks.
#include "common.cuh"
#include "internal.cuh"

namespace bsx {

constexpr int kSsThreads = 1024;
constexpr int kSsWarps = kSsThreads / 32;
constexpr int kSsSlice = 32768;   // floats of output per block
constexpr int kSsList = 2048;     // active rows listed per round (row, start, length: 16 bytes each)
constexpr int kSsUnroll = 3;      // 128-bit loads in flight per lane and array
constexpr int kSsDeal = 12;       // 32-entry stretches in flight per warp over the sliced layout

// Adds into slot `cc` of the slice at shared address `sbase` when cc < ncol.  The test is a predicate
// on the atomic itself: written as a C++ `if` around an asm statement it becomes a divergent branch
// with its convergence barrier — three more instructions per add than the add itself.
// COUNT (homogeneous weights, event input): the slice holds integer hit counts, added with the
// native shared-memory integer atomic (the float add is a load + compare-and-swap loop), and
// is multiplied by the weight once when it is written out.
// FIXED: the slot holds a signed 32-bit fixed-point sum; v arrives already scaled by 2^s.  Integer
// addition is associative, so the result does not depend on the order of the adds.
__device__ __forceinline__ void smem_red_s32_if(uint32_t sbase, uint32_t cc, uint32_t ncol, int32_t q) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.lt.u32 p, %1, %2;\n\t@p red.shared.add.s32 [%0], %3;\n\t}"
               ::"r"(sbase + (cc << 2)), "r"(cc), "r"(ncol), "r"(q) : "memory");
}
__device__ __forceinline__ void smem_count_if(uint32_t sbase, uint32_t cc, uint32_t ncol) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.lt.u32 p, %1, %2;\n\t@p red.shared.add.u32 [%0], 1;\n\t}"
               ::"r"(sbase + (cc << 2)), "r"(cc), "r"(ncol) : "memory");
}
__device__ __forceinline__ void smem_red_f32_if(uint32_t sbase, uint32_t cc, uint32_t ncol, float v) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.lt.u32 p, %1, %2;\n\t@p red.shared.add.f32 [%0], %3;\n\t}"
               ::"r"(sbase + (cc << 2)), "r"(cc), "r"(ncol), "f"(v) : "memory");
}
template <bool COUNT, bool FIXED = false>
__device__ __forceinline__ void smem_add_if(uint32_t sbase, uint32_t cc, uint32_t ncol, float v) {
  if (COUNT) smem_count_if(sbase, cc, ncol);
  else if (FIXED) smem_red_s32_if(sbase, cc, ncol, __float2int_rn(v));
  else smem_red_f32_if(sbase, cc, ncol, v);
}

// Active spikes among the positions [i0, i1) of batch row b; their positions go to dst
// when it is not null.  i0 is a multiple of 32.
template <int FORMAT>
__device__ __forceinline__ int list_span(const void* __restrict__ spikes, int64_t b, int64_t n_pre, int64_t words,
                                         int64_t i0, int64_t i1, int32_t* dst) {
  int c = 0;
  if (i0 >= i1) return 0;
  if (FORMAT == BSX_SPK_BITS32) {
    const uint32_t* __restrict__ wp = static_cast<const uint32_t*>(spikes) + b * words;
    for (int64_t k = i0 >> 5; k < ((i1 + 31) >> 5); ++k) {
      uint32_t wd = __ldg(wp + k);
      while (wd) {
        const int64_t i = (k << 5) + (__ffs(wd) - 1);
        wd &= wd - 1;
        if (i < i1) {
          if (dst) dst[c] = (int32_t)i;
          ++c;
        }
      }
    }
  } else if (FORMAT == BSX_SPK_BOOL8) {
    const uint8_t* __restrict__ sp = static_cast<const uint8_t*>(spikes) + b * n_pre;
    int64_t i = i0;
    for (; i < i1 && ((reinterpret_cast<uintptr_t>(sp + i) & 3) != 0); ++i)
      if (sp[i]) { if (dst) dst[c] = (int32_t)i; ++c; }
    for (; i + 4 <= i1; i += 4) {
      const uint32_t wd = __ldg(reinterpret_cast<const uint32_t*>(sp + i));
      if (wd == 0) continue;
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if ((wd >> (8 * k)) & 0xffu) { if (dst) dst[c] = (int32_t)(i + k); ++c; }
    }
    for (; i < i1; ++i)
      if (sp[i]) { if (dst) dst[c] = (int32_t)i; ++c; }
  } else {
    const float* __restrict__ fp = static_cast<const float*>(spikes) + b * n_pre;
    for (int64_t i = i0; i < i1; ++i)
      if (__ldg(fp + i) != 0.0f) { if (dst) dst[c] = (int32_t)i; ++c; }
  }
  return c;
}

template <bool HETERO, bool COUNT>
__device__ __forceinline__ void add_four(uint32_t sbase, int32_t col0, uint32_t ncol, const int4 j, const float4 t, float v) {
  smem_add_if<COUNT>(sbase, (uint32_t)(j.x - col0), ncol, HETERO ? __fmul_rn(v, t.x) : v);
  smem_add_if<COUNT>(sbase, (uint32_t)(j.y - col0), ncol, HETERO ? __fmul_rn(v, t.y) : v);
  smem_add_if<COUNT>(sbase, (uint32_t)(j.z - col0), ncol, HETERO ? __fmul_rn(v, t.z) : v);
  smem_add_if<COUNT>(sbase, (uint32_t)(j.w - col0), ncol, HETERO ? __fmul_rn(v, t.w) : v);
}

// PACKED (over the sliced layout only): `idx` holds 16-bit column offsets inside the slice and, for
// heterogeneous weights, `w` holds the weights already in fixed point (int32, scaled by 2^s): six
// bytes per synapse instead of eight (two instead of four for homogeneous weights), and no
// subtraction, multiplication or conversion per event.
template <bool HETERO, bool HAS_X, int FORMAT, bool SLICED, bool FIXED = false, bool PACKED = false>
__global__ void __launch_bounds__(kSsThreads, 1)
scatter_smem_kernel(RowMap rm, const int32_t* __restrict__ idx, const float* __restrict__ w,
                    const void* __restrict__ spikes, const float* __restrict__ x, int64_t n_pre,
                    int64_t n_post, float* __restrict__ out, int accumulate, bool vec_ok, int row_mul,
                    float scale = 1.0f, float inv_scale = 1.0f) {
  constexpr bool COUNT = !HETERO && !HAS_X;     // every event adds the same value: count, multiply once
  extern __shared__ __align__(16) unsigned char ss_raw[];
  float* acc = reinterpret_cast<float*>(ss_raw);
  const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(acc);
  // per listed row: where its entries start, how many there are, and which row it is
  int64_t* row_start = reinterpret_cast<int64_t*>(ss_raw + sizeof(float) * kSsSlice);
  int32_t* row_len = reinterpret_cast<int32_t*>(row_start + kSsList);
  int32_t* list = row_len + kSsList;
  __shared__ int32_t warp_tot[kSsWarps];
  __shared__ int32_t s_next;
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  // Over the sliced layout the blocks of one slice are neighbours in launch order (grid x = spike
  // vector, y = slice): the blocks resident together then read groups of the same half of the
  // matrix, whose working set (about 130 MB at 65 536 x 655) the L2 nearly holds, so the rows that
  // several vectors share are found there.  Over unsliced rows both blocks of a vector read the same
  // rows, so there the two slices of a vector are neighbours (x = slice, y = spike vector).
  const int64_t b = SLICED ? blockIdx.x : blockIdx.y;
  const int slice_id = SLICED ? (int)blockIdx.y : (int)blockIdx.x;
  const int32_t col0 = (int32_t)slice_id * kSsSlice;
  const uint32_t ncol = (uint32_t)((n_post - col0) < kSsSlice ? (n_post - col0) : kSsSlice);
  for (int i = tid; i < kSsSlice / 4; i += kSsThreads) reinterpret_cast<float4*>(acc)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  const float w0 = HETERO ? 1.0f : __ldg(w);
  const int64_t words = (n_pre + 31) >> 5;
  const int4* __restrict__ idx4 = reinterpret_cast<const int4*>(idx);
  const float4* __restrict__ w4 = reinterpret_cast<const float4*>(w);

  int64_t span = n_pre;      // first try: all active rows of the vector in one round
  int64_t lo = 0;
  while (lo < n_pre) {
    const int64_t hi = (n_pre - lo) < span ? n_pre : lo + span;
    const int64_t per = (((hi - lo + kSsThreads - 1) / kSsThreads) + 31) & ~int64_t(31);
    const int64_t i0 = lo + (int64_t)tid * per;
    const int64_t i1 = (hi - i0) < per ? hi : i0 + per;
    // ---- count, block-wide exclusive scan.  Byte spikes in aligned 64-neuron portions are held
    // in registers (four 128-bit loads in flight at once) for both the count and the write.
    uint32_t rw[16];
    bool in_regs = false;
    int c;
    if (FORMAT == BSX_SPK_BOOL8 && (per == 64 || per == 32) && i0 + per <= hi &&
        ((reinterpret_cast<uintptr_t>(static_cast<const uint8_t*>(spikes) + b * n_pre + i0) & 15) == 0)) {
      in_regs = true;
      const uint4* __restrict__ sp4 = reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(spikes) + b * n_pre + i0);
      c = 0;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const uint4 t = (16 * k < per) ? __ldg(sp4 + k) : make_uint4(0u, 0u, 0u, 0u);
        rw[4 * k + 0] = __vcmpne4(t.x, 0u) & 0x01010101u;
        rw[4 * k + 1] = __vcmpne4(t.y, 0u) & 0x01010101u;
        rw[4 * k + 2] = __vcmpne4(t.z, 0u) & 0x01010101u;
        rw[4 * k + 3] = __vcmpne4(t.w, 0u) & 0x01010101u;
      }
#pragma unroll
      for (int k = 0; k < 16; ++k) c += __popc(rw[k]);
    } else {
      c = list_span<FORMAT>(spikes, b, n_pre, words, i0, i1, nullptr);
    }
    int incl = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    if (lane == 31) warp_tot[wid] = incl;
    __syncthreads();
    int base = incl - c, total = 0;
#pragma unroll 8
    for (int k = 0; k < kSsWarps; ++k) {
      const int t = warp_tot[k];
      if (k < wid) base += t;
      total += t;
    }
    if (total > kSsList) {
      // too many for the list (only with span > kSsList: a span of kSsList neurons always fits).
      // Take spans that would hold about 0.9 lists at this density, halve on a further miss.
      int64_t next = ((hi - lo) * (kSsList - kSsList / 10) / total) & ~int64_t(1023);
      if (next > span / 2) next = (span / 2) & ~int64_t(1023);
      span = next < kSsList ? kSsList : next;
      __syncthreads();
      continue;
    }
    if (c) {
      if (in_regs) {
        int32_t* dst = list + base;
#pragma unroll
        for (int k = 0; k < 16; ++k) {
          uint32_t m = rw[k];
          while (m) {
            *dst++ = (int32_t)(i0 + 4 * k + ((__ffs(m) - 1) >> 3));
            m &= m - 1;
          }
        }
      } else {
        list_span<FORMAT>(spikes, b, n_pre, words, i0, i1, list + base);
      }
    }
    if (tid == 0) s_next = 0;
    __syncthreads();
    // ---- the ranges of all listed rows in one round trip, instead of one per row later.
    // Rows grouped by output slice: group (row, slice) is row `row * slices + slice` of the map.
    for (int t = tid; t < total; t += kSsThreads) {
      const int64_t row = list[t];
      int64_t s, e;
      rm.range(SLICED ? row * row_mul + slice_id : row, s, e);
      row_start[t] = s;
      row_len[t] = (int32_t)(e - s);
    }
    __syncthreads();
    const bool sparse_input = (int64_t)total * 32 <= hi - lo;
    // ---- warps take listed rows one at a time
    for (;;) {
      // (compressed layout, one weight: a group costs 12 registers, so a warp takes two at a time)
      constexpr int kTake = (SLICED && PACKED && !HETERO) ? 2 : 1;
      int t = 0;
      if (lane == 0) t = atomicAdd(&s_next, kTake);
      t = __shfl_sync(0xffffffffu, t, 0);
      if (t >= total) break;
      if (SLICED && kTake == 1 && sparse_input) {
        // Prefetch into L2 the group that is handed out one round of the block's warps from now:
        // no register is held while it flies, and the warp that takes it finds it a short trip away.
        // One 128-byte line per lane.
        // (Only below about 3 % of active rows: above, other vectors' blocks have brought most rows
        // into L2 already and the prefetches only add requests — 8 % slower at 10 %.)
        const int tp = t + kSsWarps;
        if (tp < total) {
          // lanes 0-15: the lines of the group's indices; lanes 16-31: those of its weights (2 KB each
          // at most, which covers 512 entries); line-aligned, so every line holds bytes of the group
          const int64_t sp = row_start[tp];
          const uint32_t lp = (uint32_t)row_len[tp];
          const bool second = lane >= 16;
          const char* base = second ? reinterpret_cast<const char*>(w) + sp * 4
                                    : reinterpret_cast<const char*>(idx) + sp * (PACKED ? 2 : 4);
          const uint32_t bytes = second ? (HETERO ? lp * 4u : 0u) : lp * (PACKED ? 2u : 4u);
          const uint32_t misal = (uint32_t)reinterpret_cast<uintptr_t>(base) & 127u;
          const uint32_t off = (uint32_t)(lane & 15) * 128u;
          if (bytes && off < misal + bytes) asm volatile("prefetch.global.L2 [%0];" ::"l"(base - misal + off));
        }
      }
      const int64_t row = list[t];
      const int64_t s = row_start[t], e = s + row_len[t];
      float v = HAS_X ? __ldg(x + b * n_pre + row) : 1.0f;
      if (!HETERO) v = __fmul_rn(v, w0);
      if (FIXED) v = __fmul_rn(v, scale);            // a power of two: exact
      if (SLICED && PACKED) {
        const uint16_t* __restrict__ gl = reinterpret_cast<const uint16_t*>(idx) + s;
        const int32_t* __restrict__ gq = reinterpret_cast<const int32_t*>(w) + s;
        const int len = row_len[t];
        if (!HETERO) {
          const bool two = t + 1 < total;
          const uint16_t* __restrict__ gl2 = reinterpret_cast<const uint16_t*>(idx) + (two ? row_start[t + 1] : s);
          const int len2 = two ? row_len[t + 1] : 0;
          const int top = len > len2 ? len : len2;
          for (int p0 = lane; p0 < top; p0 += 32 * kSsDeal) {
            uint32_t cc[kSsDeal], c2[kSsDeal];
#pragma unroll
            for (int u = 0; u < kSsDeal; ++u) {
              cc[u] = p0 + 32 * u < len ? (uint32_t)__ldg(gl + p0 + 32 * u) : 0xffffu;
              c2[u] = p0 + 32 * u < len2 ? (uint32_t)__ldg(gl2 + p0 + 32 * u) : 0xffffu;
            }
#pragma unroll
            for (int u = 0; u < kSsDeal; ++u) {
              smem_count_if(sbase, cc[u], ncol);
              smem_count_if(sbase, c2[u], ncol);
            }
          }
          continue;
        }
        for (int p0 = lane; p0 < len; p0 += 32 * kSsDeal) {
          uint32_t cc[kSsDeal];
          int32_t q[kSsDeal];
#pragma unroll
          for (int u = 0; u < kSsDeal; ++u) {
            const bool in = p0 + 32 * u < len;
            cc[u] = in ? (uint32_t)__ldg(gl + p0 + 32 * u) : 0xffffu;
            q[u] = in ? __ldg(gq + p0 + 32 * u) : 0;
          }
#pragma unroll
          for (int u = 0; u < kSsDeal; ++u) smem_red_s32_if(sbase, cc[u], ncol, q[u]);
        }
        continue;
      }
      if (SLICED) {
        // the group is laid out in 32-entry stretches whose entries fall into distinct banks:
        // one coalesced 4-byte load per lane and stretch, all issued before the first add
        // (32-bit offsets from the group's start: one 64-bit address per array and group)
        const int32_t* __restrict__ gi = idx + s;
        const float* __restrict__ gw = w + s;
        const int len = row_len[t];
        for (int p0 = lane; p0 < len; p0 += 32 * kSsDeal) {
          int32_t j[kSsDeal];
          float t[kSsDeal];
#pragma unroll
          for (int u = 0; u < kSsDeal; ++u) {
            const bool in = p0 + 32 * u < len;
            j[u] = in ? __ldg(gi + p0 + 32 * u) : -1;
            t[u] = (HETERO && in) ? __ldg(gw + p0 + 32 * u) : 0.0f;
          }
#pragma unroll
          for (int u = 0; u < kSsDeal; ++u)
            smem_add_if<COUNT, FIXED>(sbase, (uint32_t)(j[u] - col0), ncol, HETERO ? __fmul_rn(v, t[u]) : v);
        }
        continue;
      }
      int64_t a0 = e, a1 = e;
      if (vec_ok) {
        a0 = (s + 3) & ~int64_t(3);
        if (a0 > e) a0 = e;
        a1 = e & ~int64_t(3);
        if (a1 < a0) a1 = a0;
      }
      // the unaligned head and tail of the row (at most 3 + 3 entries with 128-bit loads allowed):
      // loaded now, applied after the body, so that they share the body's first round trip
      const int nh = (int)(a0 - s), nt = (int)(e - a1);
      int32_t hj = -1;
      float hw = 0.0f;
      if (vec_ok && lane < nh + nt) {
        const int64_t p = lane < nh ? s + lane : a1 + (lane - nh);
        hj = __ldg(idx + p);
        if (HETERO) hw = __ldg(w + p);
      }
      // 128-bit body: every load of a stretch is issued before its first use
      const int64_t q1 = a1 >> 2;
      for (int64_t q = (a0 >> 2) + lane; q < q1; q += 32 * kSsUnroll) {
        int4 j[kSsUnroll];
        float4 t4[kSsUnroll];
#pragma unroll
        for (int u = 0; u < kSsUnroll; ++u) {
          const bool in = q + 32 * u < q1;
          j[u] = in ? __ldg(idx4 + q + 32 * u) : make_int4(-1, -1, -1, -1);
          if (HETERO) t4[u] = in ? __ldg(w4 + q + 32 * u) : make_float4(0.f, 0.f, 0.f, 0.f);
          else t4[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int u = 0; u < kSsUnroll; ++u) add_four<HETERO, COUNT>(sbase, col0, ncol, j[u], t4[u], v);
      }
      if (vec_ok) {
        smem_add_if<COUNT>(sbase, (uint32_t)(hj - col0), ncol, HETERO ? __fmul_rn(v, hw) : v);
      } else {
        for (int64_t p = s + lane; p < e; p += 32)
          smem_add_if<COUNT>(sbase, (uint32_t)(__ldg(idx + p) - col0), ncol, HETERO ? __fmul_rn(v, __ldg(w + p)) : v);
      }
    }
    __syncthreads();
    lo = hi;
  }
  // ---- write the slice (hit counts become count * weight here, rounded once)
  float* __restrict__ ob = out + b * n_post + col0;
  auto value = [&](float slot) {
    if (COUNT) return __fmul_rn(__uint2float_rn(__float_as_uint(slot)), w0);
    if (FIXED) return __fmul_rn(__int2float_rn(__float_as_int(slot)), inv_scale);
    return slot;
  };
  if (((reinterpret_cast<uintptr_t>(ob) & 15) == 0) && (ncol % 4 == 0)) {
    float4* o4 = reinterpret_cast<float4*>(ob);
    const float4* a4 = reinterpret_cast<const float4*>(acc);
    for (int i = tid; i < (int)(ncol / 4); i += kSsThreads) {
      float4 r = a4[i];
      r.x = value(r.x); r.y = value(r.y); r.z = value(r.z); r.w = value(r.w);
      if (accumulate) {
        const float4 old = o4[i];
        r.x += old.x; r.y += old.y; r.z += old.z; r.w += old.w;
      }
      o4[i] = r;
    }
  } else {
    for (int i = tid; i < (int)ncol; i += kSsThreads) ob[i] = accumulate ? ob[i] + value(acc[i]) : value(acc[i]);
  }
}

// Groups the entries of every row by output slice (slice = column / 32768).
// s_indptr[row * S + k] is where group k of the row starts; the row keeps its place
// [start, end) in the arrays.  Inside a group the entries are laid out for the scatter
// kernel, whose warps read 32 consecutive entries per instruction and add them to shared
// memory: the group is sorted by shared-memory bank (column mod 32, original order kept
// inside a bank) and dealt round-robin over its 32-entry stretches, so that the entries
// of one stretch fall into distinct banks as far as the group allows.  Entry number k of
// the bank-sorted group of n entries, J = ceil(n / 32) stretches, the last one holding
// m = n - 32 (J - 1):  k < m J  ->  stretch k mod J, slot k div J;  otherwise, with
// k' = k - m J:  stretch k' mod (J - 1), slot m + k' div (J - 1).
// With s_indices == nullptr only the offsets are written (for rows that are already
// grouped, e.g. sorted by column).  One warp per row.  Columns beyond the last slice
// are kept in the last group.
constexpr int kSliceWarps = 8;

__device__ __forceinline__ uint32_t slice_key(int32_t col, int S) {
  uint32_t sl = (uint32_t)col / (uint32_t)kSsSlice;
  if (sl > (uint32_t)(S - 1)) sl = (uint32_t)(S - 1);
  return sl * 32u + ((uint32_t)col & 31u);
}

__global__ void __launch_bounds__(kSliceWarps * 32)
slice_rows_kernel(RowMap rm, const int32_t* __restrict__ idx, int64_t n_pre, int S, int64_t nnz,
                  int64_t* __restrict__ s_indptr, int32_t* __restrict__ s_indices, int32_t* __restrict__ s_perm) {
  __shared__ int32_t hist_all[kSliceWarps][128];
  const int lane = threadIdx.x & 31;
  int32_t* hist = hist_all[threadIdx.x >> 5];
  const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const uint32_t lt = (1u << lane) - 1u;
  if (warp == 0 && lane == 0) s_indptr[n_pre * S] = nnz;
  for (int64_t row = warp; row < n_pre; row += nwarps) {
    int64_t s, e;
    rm.range(row, s, e);
    // entries per (slice, bank)
#pragma unroll
    for (int k = 0; k < 4; ++k) hist[32 * k + lane] = 0;
    __syncwarp();
    for (int64_t p = s + lane; p < e; p += 32) atomicAdd(&hist[slice_key(__ldg(idx + p), S)], 1);
    __syncwarp();
    // group sizes and starts; hist becomes the running start of every bank inside its group
    int n[4];
    int64_t base[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int c = hist[32 * k + lane];
      int incl = c;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
      }
      n[k] = __shfl_sync(0xffffffffu, incl, 31);
      hist[32 * k + lane] = incl - c;
    }
    base[0] = s;
#pragma unroll
    for (int k = 1; k < 4; ++k) base[k] = base[k - 1] + n[k - 1];
    if (lane < S) s_indptr[row * S + lane] = lane == 0 ? base[0] : lane == 1 ? base[1] : lane == 2 ? base[2] : base[3];
    __syncwarp();
    if (!s_indices) continue;
    for (int64_t p0 = s; p0 < e; p0 += 32) {
      const int64_t p = p0 + lane;
      int32_t col = 0;
      uint32_t key = 0xffffffffu;
      if (p < e) {
        col = __ldg(idx + p);
        key = slice_key(col, S);
      }
      const uint32_t same = __match_any_sync(0xffffffffu, key);
      int k_sorted = 0;
      if (p < e) k_sorted = hist[key] + __popc(same & lt);
      __syncwarp();
      if (p < e && (same & lt) == 0) hist[key] += __popc(same);    // the first lane of every key moves it on
      __syncwarp();
      if (p < e) {
        const int sl = (int)(key >> 5);
        const int ng = sl == 0 ? n[0] : sl == 1 ? n[1] : sl == 2 ? n[2] : n[3];
        const int64_t gb = sl == 0 ? base[0] : sl == 1 ? base[1] : sl == 2 ? base[2] : base[3];
        const int J = (ng + 31) >> 5;
        const int m = ng - 32 * (J - 1);
        int stretch, slot;
        if (k_sorted < m * J) {
          stretch = k_sorted % J;
          slot = k_sorted / J;
        } else {
          const int k2 = k_sorted - m * J;
          stretch = k2 % (J - 1);
          slot = m + k2 / (J - 1);
        }
        const int64_t pos = gb + 32 * stretch + slot;
        s_indices[pos] = col;
        s_perm[pos] = (int32_t)p;
      }
    }
    __syncwarp();
  }
}

bool scatter_smem_applies(const bsx_conn_t* conn, int format, int64_t batch) {
  if (format != BSX_SPK_BOOL8 && format != BSX_SPK_F32 && format != BSX_SPK_BITS32) return false;
  const int64_t slices = (conn->n_post + kSsSlice - 1) / kSsSlice;
  return batch >= 16 && batch <= 65535 && slices >= 1 && slices <= 4;
}

bool scatter_smem_preferred(const bsx_conn_t* conn, int format, int64_t batch) {
  if (!scatter_smem_applies(conn, format, batch)) return false;
  const int64_t slices = (conn->n_post + kSsSlice - 1) / kSsSlice;
  const int sms = sm_count();
  return sms > 0 && slices <= 2 && batch * slices * 4 >= (int64_t)sms * 3;
}

// Deterministic form over the sliced layout: heterogeneous weights summed in 2^-scale_log2 fixed point.
static int launch_scatter_smem_fixed(const bsx_conn_t* conn, const void* spikes, int format, int64_t batch, float* out,
                                     int accumulate, cudaStream_t st, int row_mul, int scale_log2) {
  if (sm_count() <= 0) return fail(BSX_ERR_CUDA, "no CUDA device");
  const int64_t slices = (conn->n_post + kSsSlice - 1) / kSsSlice;
  const dim3 grid((unsigned)batch, (unsigned)slices, 1);      // sliced layout: x = spike vector, y = slice
  const size_t smem = sizeof(float) * kSsSlice + (sizeof(int64_t) + 2 * sizeof(int32_t)) * kSsList;
  const bool vec_ok = aligned16(conn->indices) && aligned16(conn->weights);
  const RowMap rm = make_rowmap(conn);
  const float scale = ldexpf(1.0f, scale_log2), inv_scale = ldexpf(1.0f, -scale_log2);
#define BSX_SSF(F)                                                                                                   \
  do {                                                                                                               \
    BSX_CUDA(cudaFuncSetAttribute(scatter_smem_kernel<true, false, F, true, true>,                                   \
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));                          \
    scatter_smem_kernel<true, false, F, true, true><<<grid, kSsThreads, smem, st>>>(                                 \
        rm, conn->indices, conn->weights, spikes, nullptr, conn->n_pre, conn->n_post, out, accumulate, vec_ok, row_mul, \
        scale, inv_scale);                                                                                           \
  } while (0)
  if (format == BSX_SPK_BOOL8) BSX_SSF(BSX_SPK_BOOL8);
  else if (format == BSX_SPK_F32) BSX_SSF(BSX_SPK_F32);
  else BSX_SSF(BSX_SPK_BITS32);
#undef BSX_SSF
  BSX_LAUNCH_CHECK("scatter_smem_kernel<fixed>");
  return BSX_OK;
}

// The same over 16-bit column offsets and (heterogeneous) weights stored in fixed point.
static int launch_scatter_smem_packed(const bsx_conn_t* conn, const uint16_t* local, const int32_t* qweights,
                                      const void* spikes, int format, int64_t batch, float* out, int accumulate,
                                      cudaStream_t st, int row_mul, int scale_log2) {
  if (sm_count() <= 0) return fail(BSX_ERR_CUDA, "no CUDA device");
  const int64_t slices = (conn->n_post + kSsSlice - 1) / kSsSlice;
  const dim3 grid((unsigned)batch, (unsigned)slices, 1);      // sliced layout: x = spike vector, y = slice
  const size_t smem = sizeof(float) * kSsSlice + (sizeof(int64_t) + 2 * sizeof(int32_t)) * kSsList;
  const RowMap rm = make_rowmap(conn);
  const float scale = ldexpf(1.0f, scale_log2), inv_scale = ldexpf(1.0f, -scale_log2);
  const int32_t* idx = reinterpret_cast<const int32_t*>(local);
  const float* w = conn->hetero ? reinterpret_cast<const float*>(qweights) : conn->weights;
#define BSX_SSP(H, F)                                                                                               \
  do {                                                                                                              \
    BSX_CUDA(cudaFuncSetAttribute(scatter_smem_kernel<H, false, F, true, H, true>,                                  \
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));                         \
    scatter_smem_kernel<H, false, F, true, H, true><<<grid, kSsThreads, smem, st>>>(                                \
        rm, idx, w, spikes, nullptr, conn->n_pre, conn->n_post, out, accumulate, false, row_mul, scale, inv_scale); \
  } while (0)
#define BSX_SSP_F(H)                                           \
  do {                                                         \
    if (format == BSX_SPK_BOOL8) BSX_SSP(H, BSX_SPK_BOOL8);    \
    else if (format == BSX_SPK_F32) BSX_SSP(H, BSX_SPK_F32);   \
    else BSX_SSP(H, BSX_SPK_BITS32);                           \
  } while (0)
  if (conn->hetero) BSX_SSP_F(true); else BSX_SSP_F(false);
#undef BSX_SSP_F
#undef BSX_SSP
  BSX_LAUNCH_CHECK("scatter_smem_kernel<packed>");
  return BSX_OK;
}

__global__ void __launch_bounds__(256)
compress_local_kernel(const int32_t* __restrict__ idx, int64_t nnz, int32_t last_slice, uint16_t* __restrict__ local) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t p = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; p < nnz; p += stride) {
    const int32_t c = __ldg(idx + p);
    // a column is stored relative to the start of its slice; negative or too large columns (which
    // bsx_validate_conn reports) get an offset no slice accepts
    const int32_t sl = c / kSsSlice;
    local[p] = (c < 0 || sl > last_slice) ? (uint16_t)0xffffu : (uint16_t)(c - sl * kSsSlice);
  }
}

__global__ void __launch_bounds__(256)
quantize_kernel(const float* __restrict__ w, int64_t n, float scale, int32_t* __restrict__ q) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t p = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; p < n; p += stride)
    q[p] = __float2int_rn(__fmul_rn(__ldg(w + p), scale));
}

// |w| summed per output column as 2^-32 fixed point (order-free), then the largest column.
__global__ void __launch_bounds__(256)
abs_sum_kernel(const int32_t* __restrict__ idx, const float* __restrict__ w, int64_t nnz,
               unsigned long long* __restrict__ col_sum) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t p = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; p < nnz; p += stride) {
    const unsigned long long q = (unsigned long long)__float2ll_rn(fabsf(__ldg(w + p)) * 4294967296.0f);
    atomicAdd(col_sum + __ldg(idx + p), q);
  }
}
__global__ void __launch_bounds__(256)
max_u64_kernel(const unsigned long long* __restrict__ v, int64_t n, unsigned long long* __restrict__ out) {
  unsigned long long m = 0;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) m = v[i] > m ? v[i] : m;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long t = __shfl_xor_sync(0xffffffffu, m, o);
    m = t > m ? t : m;
  }
  if ((threadIdx.x & 31) == 0 && m) atomicMax(out, m);
}

int launch_scatter_smem(const bsx_conn_t* conn, const void* spikes, int format, const float* x, int64_t batch,
                        float* out, int accumulate, cudaStream_t st, int row_mul) {
  if (sm_count() <= 0) return fail(BSX_ERR_CUDA, "no CUDA device");
  const int64_t slices = (conn->n_post + kSsSlice - 1) / kSsSlice;
  const dim3 grid = row_mul >= 1 ? dim3((unsigned)batch, (unsigned)slices, 1)       // sliced: x = spike vector, y = slice
                                 : dim3((unsigned)slices, (unsigned)batch, 1);
  const size_t smem = sizeof(float) * kSsSlice + (sizeof(int64_t) + 2 * sizeof(int32_t)) * kSsList;
  const bool vec_ok = aligned16(conn->indices) && (!conn->hetero || aligned16(conn->weights));
  const RowMap rm = make_rowmap(conn);
#define BSX_SS2(H, X, F, SL)                                                                                    \
  do {                                                                                                          \
    BSX_CUDA(cudaFuncSetAttribute(scatter_smem_kernel<H, X, F, SL>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                  (int)smem));                                                                  \
    scatter_smem_kernel<H, X, F, SL><<<grid, kSsThreads, smem, st>>>(rm, conn->indices, conn->weights, spikes,  \
                                                                     x, conn->n_pre, conn->n_post, out,         \
                                                                     accumulate, vec_ok, row_mul);              \
  } while (0)
#define BSX_SS(H, X, F)                          \
  do {                                           \
    if (row_mul >= 1) BSX_SS2(H, X, F, true);    \
    else BSX_SS2(H, X, F, false);                \
  } while (0)
#define BSX_SS_F(H, X)                                           \
  do {                                                           \
    if (format == BSX_SPK_BOOL8) BSX_SS(H, X, BSX_SPK_BOOL8);    \
    else if (format == BSX_SPK_F32) BSX_SS(H, X, BSX_SPK_F32);   \
    else BSX_SS(H, X, BSX_SPK_BITS32);                           \
  } while (0)
  if (conn->hetero) {
    if (x) BSX_SS_F(true, true); else BSX_SS_F(true, false);
  } else {
    if (x) BSX_SS_F(false, true); else BSX_SS_F(false, false);
  }
#undef BSX_SS_F
#undef BSX_SS
#undef BSX_SS2
  BSX_LAUNCH_CHECK("scatter_smem_kernel");
  return BSX_OK;
}

}  // namespace bsx

using namespace bsx;

extern "C" {

int64_t bsx_sliced_slices(int64_t n_post) { return n_post <= 0 ? 0 : (n_post + kSsSlice - 1) / kSsSlice; }

int bsx_sliced_build(const bsx_conn_t* conn, int64_t* s_indptr, int32_t* s_indices, int32_t* s_perm,
                     bsx_stream_t stream) {
  BSX_TRACE("bsx_sliced_build");
  const int rc = check_conn(conn);
  if (rc) return rc;
  const int64_t S = bsx_sliced_slices(conn->n_post);
  if (S < 1 || S > 4) return fail(BSX_ERR_UNSUPPORTED, "the sliced layout covers 1 to 131072 columns");
  if (!s_indptr) return fail(BSX_ERR_INVALID_ARG, "s_indptr is NULL");
  if ((s_indices == nullptr) != (s_perm == nullptr))
    return fail(BSX_ERR_INVALID_ARG, "s_indices and s_perm are given together or not at all");
  if (conn->nnz >= (int64_t)INT32_MAX) return fail(BSX_ERR_UNSUPPORTED, "nnz must be below 2^31");
  const int sms = sm_count();
  if (sms <= 0) return fail(BSX_ERR_CUDA, "no CUDA device");
  int64_t blocks = (conn->n_pre + kSliceWarps - 1) / kSliceWarps;
  if (blocks < 1) blocks = 1;
  if (blocks > (int64_t)sms * 16) blocks = (int64_t)sms * 16;
  slice_rows_kernel<<<(unsigned)blocks, kSliceWarps * 32, 0, as_stream(stream)>>>(make_rowmap(conn), conn->indices, conn->n_pre,
                                                                     (int)S, conn->nnz, s_indptr, s_indices, s_perm);
  BSX_LAUNCH_CHECK("slice_rows_kernel");
  return BSX_OK;
}

int bsx_event_vecmat_sliced(const bsx_conn_t* sliced, const void* spikes, int spike_format, int64_t batch,
                            float* out, int accumulate, bsx_stream_t stream) {
  BSX_TRACE("bsx_event_vecmat_sliced");
  const int rc = check_conn(sliced);
  if (rc) return rc;
  if (!sliced->indptr || !sliced->indptr_is_64)
    return fail(BSX_ERR_INVALID_ARG, "the sliced layout has 64-bit group offsets in indptr");
  if (batch < 0) return fail(BSX_ERR_INVALID_ARG, "negative batch");
  if (batch == 0 || sliced->n_post == 0) return BSX_OK;
  if (!out) return fail(BSX_ERR_INVALID_ARG, "out is NULL");
  if (sliced->n_pre == 0) return accumulate ? BSX_OK : launch_zero(out, batch * sliced->n_post, as_stream(stream));
  if (!spikes) return fail(BSX_ERR_INVALID_ARG, "input vector is NULL");
  if (spike_format != BSX_SPK_BOOL8 && spike_format != BSX_SPK_F32 && spike_format != BSX_SPK_BITS32)
    return fail(BSX_ERR_UNSUPPORTED, "the sliced scatter takes byte, float or packed spikes");
  const int64_t S = bsx_sliced_slices(sliced->n_post);
  if (S > 4 || batch > 65535) return fail(BSX_ERR_UNSUPPORTED, "the sliced scatter covers up to 131072 columns and 65535 vectors");
  return launch_scatter_smem(sliced, spikes, spike_format, nullptr, batch, out, accumulate, as_stream(stream), (int)S);
}

size_t bsx_fixed_scale_workspace_bytes(int64_t n_post) {
  return n_post < 0 ? 0 : ((size_t)(n_post + 1) * sizeof(unsigned long long) + 255) & ~size_t(255);
}

int bsx_fixed_scale_log2(const bsx_conn_t* conn, void* workspace, size_t workspace_bytes, int32_t* host_scale_log2,
                         bsx_stream_t stream) {
  BSX_TRACE("bsx_fixed_scale_log2");
  const int rc = check_conn(conn);
  if (rc) return rc;
  if (!host_scale_log2) return fail(BSX_ERR_INVALID_ARG, "host_scale_log2 is NULL");
  *host_scale_log2 = 0;
  if (!conn->hetero || conn->nnz == 0 || conn->n_post == 0) return BSX_OK;     // counted, not summed: nothing to scale
  const size_t need = bsx_fixed_scale_workspace_bytes(conn->n_post);
  if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 7) || workspace_bytes < need)
    return fail(BSX_ERR_WORKSPACE, "bsx_fixed_scale_log2 needs %zu workspace bytes", need);
  const int sms = sm_count();
  if (sms <= 0) return fail(BSX_ERR_CUDA, "no CUDA device");
  cudaStream_t st = as_stream(stream);
  unsigned long long* col = static_cast<unsigned long long*>(workspace);
  BSX_CUDA(cudaMemsetAsync(col, 0, need, st));
  abs_sum_kernel<<<(unsigned)(sms * 8), 256, 0, st>>>(conn->indices, conn->weights, conn->nnz, col);
  BSX_LAUNCH_CHECK("abs_sum_kernel");
  max_u64_kernel<<<(unsigned)(sms * 2), 256, 0, st>>>(col, conn->n_post, col + conn->n_post);
  BSX_LAUNCH_CHECK("max_u64_kernel");
  unsigned long long host_max = 0;
  BSX_CUDA(cudaMemcpyAsync(&host_max, col + conn->n_post, sizeof(host_max), cudaMemcpyDeviceToHost, st));
  BSX_CUDA(cudaStreamSynchronize(st));
  // the largest |sum| any output can reach is host_max * 2^-32; keep it below 2^30 after scaling
  double bound = (double)host_max / 4294967296.0;
  int s = 30;
  if (bound > 0.0) {
    s = (int)floor(log2(1073741824.0 / bound));
    if (s > 30) s = 30;
    if (s < -60) s = -60;
  }
  *host_scale_log2 = s;
  return BSX_OK;
}

int bsx_event_vecmat_sliced_fixed(const bsx_conn_t* sliced, const void* spikes, int spike_format, int64_t batch,
                                  float* out, int accumulate, int32_t scale_log2, bsx_stream_t stream) {
  BSX_TRACE("bsx_event_vecmat_sliced_fixed");
  const int rc = check_conn(sliced);
  if (rc) return rc;
  if (!sliced->hetero)        // homogeneous weights are counted as integers already: order-free as it is
    return bsx_event_vecmat_sliced(sliced, spikes, spike_format, batch, out, accumulate, stream);
  if (!sliced->indptr || !sliced->indptr_is_64)
    return fail(BSX_ERR_INVALID_ARG, "the sliced layout has 64-bit group offsets in indptr");
  if (batch < 0) return fail(BSX_ERR_INVALID_ARG, "negative batch");
  if (scale_log2 < -60 || scale_log2 > 30) return fail(BSX_ERR_INVALID_ARG, "scale_log2 out of range (see bsx_fixed_scale_log2)");
  if (batch == 0 || sliced->n_post == 0) return BSX_OK;
  if (!out) return fail(BSX_ERR_INVALID_ARG, "out is NULL");
  if (sliced->n_pre == 0) return accumulate ? BSX_OK : launch_zero(out, batch * sliced->n_post, as_stream(stream));
  if (!spikes) return fail(BSX_ERR_INVALID_ARG, "input vector is NULL");
  if (spike_format != BSX_SPK_BOOL8 && spike_format != BSX_SPK_F32 && spike_format != BSX_SPK_BITS32)
    return fail(BSX_ERR_UNSUPPORTED, "the sliced scatter takes byte, float or packed spikes");
  const int64_t S = bsx_sliced_slices(sliced->n_post);
  if (S > 4 || batch > 65535) return fail(BSX_ERR_UNSUPPORTED, "the sliced scatter covers up to 131072 columns and 65535 vectors");
  return launch_scatter_smem_fixed(sliced, spikes, spike_format, batch, out, accumulate, as_stream(stream), (int)S,
                                   scale_log2);
}

int bsx_sliced_compress(const bsx_conn_t* sliced, uint16_t* local, bsx_stream_t stream) {
  BSX_TRACE("bsx_sliced_compress");
  const int rc = check_conn(sliced);
  if (rc) return rc;
  const int64_t S = bsx_sliced_slices(sliced->n_post);
  if (S < 1 || S > 4) return fail(BSX_ERR_UNSUPPORTED, "the sliced layout covers 1 to 131072 columns");
  if (sliced->nnz == 0) return BSX_OK;
  if (!local) return fail(BSX_ERR_INVALID_ARG, "local is NULL");
  const int sms = sm_count();
  if (sms <= 0) return fail(BSX_ERR_CUDA, "no CUDA device");
  compress_local_kernel<<<(unsigned)(sms * 8), 256, 0, as_stream(stream)>>>(sliced->indices, sliced->nnz, (int32_t)(S - 1), local);
  BSX_LAUNCH_CHECK("compress_local_kernel");
  return BSX_OK;
}

int bsx_quantize_f32(const float* w, int64_t n, int32_t scale_log2, int32_t* q, bsx_stream_t stream) {
  BSX_TRACE("bsx_quantize_f32");
  if (n < 0) return fail(BSX_ERR_INVALID_ARG, "negative n");
  if (scale_log2 < -60 || scale_log2 > 30) return fail(BSX_ERR_INVALID_ARG, "scale_log2 out of range (see bsx_fixed_scale_log2)");
  if (n == 0) return BSX_OK;
  if (!w || !q) return fail(BSX_ERR_INVALID_ARG, "w or q is NULL");
  const int sms = sm_count();
  if (sms <= 0) return fail(BSX_ERR_CUDA, "no CUDA device");
  quantize_kernel<<<(unsigned)(sms * 8), 256, 0, as_stream(stream)>>>(w, n, ldexpf(1.0f, scale_log2), q);
  BSX_LAUNCH_CHECK("quantize_kernel");
  return BSX_OK;
}

int bsx_event_vecmat_sliced16(const bsx_conn_t* sliced, const uint16_t* local, const int32_t* qweights,
                              const void* spikes, int spike_format, int64_t batch, float* out, int accumulate,
                              int32_t scale_log2, bsx_stream_t stream) {
  BSX_TRACE("bsx_event_vecmat_sliced16");
  const int rc = check_conn(sliced);
  if (rc) return rc;
  if (!sliced->indptr || !sliced->indptr_is_64)
    return fail(BSX_ERR_INVALID_ARG, "the sliced layout has 64-bit group offsets in indptr");
  if (batch < 0) return fail(BSX_ERR_INVALID_ARG, "negative batch");
  if (scale_log2 < -60 || scale_log2 > 30) return fail(BSX_ERR_INVALID_ARG, "scale_log2 out of range (see bsx_fixed_scale_log2)");
  if (batch == 0 || sliced->n_post == 0) return BSX_OK;
  if (!out) return fail(BSX_ERR_INVALID_ARG, "out is NULL");
  if (sliced->n_pre == 0 || sliced->nnz == 0)
    return accumulate ? BSX_OK : launch_zero(out, batch * sliced->n_post, as_stream(stream));
  if (!spikes) return fail(BSX_ERR_INVALID_ARG, "input vector is NULL");
  if (!local) return fail(BSX_ERR_INVALID_ARG, "local is NULL");
  if (sliced->hetero && !qweights) return fail(BSX_ERR_INVALID_ARG, "heterogeneous weights need qweights (bsx_quantize_f32)");
  if ((reinterpret_cast<uintptr_t>(local) & 1) || (reinterpret_cast<uintptr_t>(qweights) & 3))
    return fail(BSX_ERR_INVALID_ARG, "local or qweights misaligned");
  if (spike_format != BSX_SPK_BOOL8 && spike_format != BSX_SPK_F32 && spike_format != BSX_SPK_BITS32)
    return fail(BSX_ERR_UNSUPPORTED, "the sliced scatter takes byte, float or packed spikes");
  const int64_t S = bsx_sliced_slices(sliced->n_post);
  if (S > 4 || batch > 65535) return fail(BSX_ERR_UNSUPPORTED, "the sliced scatter covers up to 131072 columns and 65535 vectors");
  return launch_scatter_smem_packed(sliced, local, qweights, spikes, spike_format, batch, out, accumulate,
                                    as_stream(stream), (int)S, scale_log2);
}

}  // extern "C"

