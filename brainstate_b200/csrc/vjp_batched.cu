// Reverse mode of y = x @ W for a batch of inputs (the training step of the batched
// event matmul): one pass over the indices produces
//   dx[b, i] = sum_k w[i,k] ct[b, idx[i,k]]                 (dense, every b)
//   dw[i, k] = sum_b a[b,i] ct[b, idx[i,k]]                 (heterogeneous)
//   dw       = sum_b sum_i a[b,i] sum_k ct[b, idx[i,k]]     (homogeneous)
// with a = x or the event indicator [x != 0].
//
// The cotangent is first transposed to batch-minor order (n_post, Bp) so that one
// index fetches the values of 64 batch lanes as one contiguous 256-byte stretch.  The input
// cotangent and the weight cotangent are separate launches: dx walks every synapse for every
// batch lane (lane = batch lane), dw only touches the batch lanes where the row was active —
// a handful at the firing rates of interest, found by ballot — with lane = synapse.  No
// atomics; fixed summation order.
#include "common.cuh"
#include "internal.cuh"

namespace bsx {

// (B, n) row-major -> (n, Bp) row-major, zero padded to Bp columns.
__global__ void __launch_bounds__(256)
transpose_pad_kernel(const float* __restrict__ src, int64_t B, int64_t n, int64_t Bp, float* __restrict__ dst) {
  __shared__ float tile[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  const int64_t n0 = (int64_t)blockIdx.x * 32, b0 = (int64_t)blockIdx.y * 32;
  for (int r = ty; r < 32; r += 8) {
    const int64_t b = b0 + r, j = n0 + tx;
    tile[r][tx] = (b < B && j < n) ? src[b * n + j] : 0.f;
  }
  __syncthreads();
  for (int r = ty; r < 32; r += 8) {
    const int64_t j = n0 + r, b = b0 + tx;
    if (j < n && b < Bp) dst[j * Bp + b] = tile[tx][r];
  }
}

int launch_transpose_pad(const float* src, int64_t B, int64_t n, int64_t Bp, float* dst, cudaStream_t st) {
  if (Bp % 32 || Bp / 32 > 65535) return fail(BSX_ERR_UNSUPPORTED, "batch too large");
  dim3 grid((unsigned)((n + 31) / 32), (unsigned)(Bp / 32), 1);
  transpose_pad_kernel<<<grid, 256, 0, st>>>(src, B, n, Bp, dst);
  BSX_LAUNCH_CHECK("transpose_pad_kernel");
  return BSX_OK;
}

template <int XFORMAT>
__device__ __forceinline__ float act_at(const void* x, int64_t pos, bool event) {
  float a = (XFORMAT == BSX_SPK_BOOL8) ? (float)(static_cast<const uint8_t*>(x)[pos] != 0)
                                       : static_cast<const float*>(x)[pos];
  if (event) a = (a != 0.f) ? 1.f : 0.f;
  return a;
}

// Input cotangent for one chunk of up to 64 batch lanes starting at b0: a warp owns a row,
// lane l holds batch lanes l and l + 32; every index fetches its 64 cotangent values as one
// 256-byte stretch of the batch-minor copy (one 8-byte load per lane).
constexpr int kDxFlight = 8;    // 128-bit loads per lane in flight = 16 cotangent stretches per warp (4: 1.3x slower, 16: 1.2x slower)

template <bool HETERO>
__global__ void __launch_bounds__(256)
vjp_dx_batched_kernel(RowMap rm, const int32_t* __restrict__ idx, const float* __restrict__ w,
                      const float* __restrict__ ctT, int64_t Bp, int64_t B, int64_t b0, int64_t n_pre,
                      float* __restrict__ dx) {
  const int lane = threadIdx.x & 31;
  const float w0 = HETERO ? 0.f : __ldg(w);
  // lane l reads the pair (2l, 2l + 1) of the 64 lanes: one float2 per lane covers the stretch
  const int64_t be = b0 + 2 * lane, bo = be + 1;
  const bool pair = b0 + 64 <= Bp;                       // a full 64-lane stretch exists
  const int half = lane >> 4, quad = lane & 15;
  const int64_t wstep = (int64_t)gridDim.x * (blockDim.x >> 5);
  for (int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < n_pre; row += wstep) {
    // the index and weight lines of the warp's next row go to L2 now (rows of a fixed length: their
    // place is known without a load): every 32-synapse stretch below starts with a load of them
    if (!rm.p64 && !rm.p32 && row + wstep < n_pre) {
      const char* fi = reinterpret_cast<const char*>(idx + (row + wstep) * rm.K);
      const char* li = fi - (reinterpret_cast<uintptr_t>(fi) & 127) + 128 * lane;
      if (li < fi + rm.K * 4) asm volatile("prefetch.global.L2 [%0];" ::"l"(li));
      if (HETERO) {
        const char* fw = reinterpret_cast<const char*>(w + (row + wstep) * rm.K);
        const char* lw = fw - (reinterpret_cast<uintptr_t>(fw) & 127) + 128 * lane;
        if (lw < fw + rm.K * 4) asm volatile("prefetch.global.L2 [%0];" ::"l"(lw));
      }
    }
    int64_t s, e;
    rm.range(row, s, e);
    float acc_e = 0.f, acc_o = 0.f;
    float4 acc4 = make_float4(0.f, 0.f, 0.f, 0.f);       // batch lanes 4 * quad .. + 3, this half-warp's synapses
    for (int64_t pb = s; pb < e; pb += 32) {
      const int64_t p = pb + lane;
      int32_t j_l = 0;
      float w_l = 0.f;
      if (p < e) {
        j_l = __ldg(idx + p);
        w_l = HETERO ? __ldg(w + p) : 1.f;
      }
      const int cnt = (int)((e - pb) < 32 ? (e - pb) : 32);
      if (pair && cnt == 32) {
        // the common case: 32 synapses.  Each half-warp takes every other synapse, one 128-bit load
        // per lane (16 lanes x 4 batch lanes = the 256-byte stretch), kDxFlight loads — 2 * kDxFlight
        // stretches per warp — requested before any is used: the kernel is bound by the latency of
        // these L2 gathers.
#pragma unroll
        for (int t0 = 0; t0 < 16; t0 += kDxFlight) {
          float4 c[kDxFlight];
#pragma unroll
          for (int u = 0; u < kDxFlight; ++u) {
            const int32_t j = __shfl_sync(0xffffffffu, j_l, 2 * (t0 + u) + half);
            c[u] = __ldg(reinterpret_cast<const float4*>(ctT + (int64_t)j * Bp + b0) + quad);
          }
#pragma unroll
          for (int u = 0; u < kDxFlight; ++u) {
            const float ww = __shfl_sync(0xffffffffu, w_l, 2 * (t0 + u) + half);
            acc4.x = fmaf(ww, c[u].x, acc4.x);
            acc4.y = fmaf(ww, c[u].y, acc4.y);
            acc4.z = fmaf(ww, c[u].z, acc4.z);
            acc4.w = fmaf(ww, c[u].w, acc4.w);
          }
        }
        continue;
      }
#pragma unroll 4
      for (int t = 0; t < cnt; ++t) {
        const int32_t j = __shfl_sync(0xffffffffu, j_l, t);
        const float ww = __shfl_sync(0xffffffffu, w_l, t);
        const float* __restrict__ crow = ctT + (int64_t)j * Bp + b0;
        float2 c;
        if (pair) c = __ldg(reinterpret_cast<const float2*>(crow) + lane);
        else c = make_float2(lane < 16 ? __ldg(crow + 2 * lane) : 0.f, lane < 16 ? __ldg(crow + 2 * lane + 1) : 0.f);
        acc_e = fmaf(ww, c.x, acc_e);
        acc_o = fmaf(ww, c.y, acc_o);
      }
    }
    // fold the 128-bit path into the pair layout: the two half-warps are summed, then lane l takes
    // batch lanes 2l and 2l + 1 from lane l / 2 (fixed order: deterministic)
    acc4.x += __shfl_xor_sync(0xffffffffu, acc4.x, 16);
    acc4.y += __shfl_xor_sync(0xffffffffu, acc4.y, 16);
    acc4.z += __shfl_xor_sync(0xffffffffu, acc4.z, 16);
    acc4.w += __shfl_xor_sync(0xffffffffu, acc4.w, 16);
    {
      const int src = lane >> 1;
      const float lo_a = __shfl_sync(0xffffffffu, acc4.x, src), lo_b = __shfl_sync(0xffffffffu, acc4.y, src);
      const float hi_a = __shfl_sync(0xffffffffu, acc4.z, src), hi_b = __shfl_sync(0xffffffffu, acc4.w, src);
      acc_e += (lane & 1) ? hi_a : lo_a;
      acc_o += (lane & 1) ? hi_b : lo_b;
    }
    if (!HETERO) { acc_e *= w0; acc_o *= w0; }
    if (be < B) dx[be * n_pre + row] = acc_e;
    if (bo < B) dx[bo * n_pre + row] = acc_o;
  }
}

// Weight cotangent for one chunk of up to 64 batch lanes starting at b0: a warp owns a row
// and first finds the batch lanes where the row was active (ballot).  With few of them (the
// event case: a handful at the firing rates of interest) lane = synapse: every lane gathers
// the cotangent of its own target for each active batch lane, in ascending batch order.  With
// many (a dense float input) lane = batch lane over the batch-minor copy and a warp sum per
// synapse.  No atomics, fixed summation order.  first_chunk: dw is written, later chunks add.
template <bool HETERO, int XFORMAT>
__global__ void __launch_bounds__(256)
vjp_dw_batched_kernel(RowMap rm, const int32_t* __restrict__ idx, const void* __restrict__ x, bool event,
                      const float* __restrict__ ct, const float* __restrict__ ctT, int64_t Bp, int64_t B, int64_t b0,
                      int64_t n_pre, int64_t n_post, float* __restrict__ dw, bool first_chunk) {
  __shared__ float block_part[8];
  const int lane = threadIdx.x & 31;
  const int64_t blo = b0 + lane, bhi = b0 + 32 + lane;
  const bool has_lo = blo < B, has_hi = bhi < B;
  float homo_acc = 0.f;
  const int64_t wstep = (int64_t)gridDim.x * (blockDim.x >> 5);
  for (int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < n_pre; row += wstep) {
    // the index lines of the warp's next row go to L2 now (rows of a fixed length: their place is
    // known without a load), so that the row's first loads do not wait for DRAM
    if (!rm.p64 && !rm.p32 && row + wstep < n_pre) {
      const char* first = reinterpret_cast<const char*>(idx + (row + wstep) * rm.K);
      const char* line = first - (reinterpret_cast<uintptr_t>(first) & 127) + 128 * lane;
      if (line < first + rm.K * 4) asm volatile("prefetch.global.L2 [%0];" ::"l"(line));
    }
    const float a_lo = has_lo ? act_at<XFORMAT>(x, blo * n_pre + row, event) : 0.f;
    const float a_hi = has_hi ? act_at<XFORMAT>(x, bhi * n_pre + row, event) : 0.f;
    const uint32_t act_lo = __ballot_sync(0xffffffffu, a_lo != 0.f);
    const uint32_t act_hi = __ballot_sync(0xffffffffu, a_hi != 0.f);
    int64_t s, e;
    rm.range(row, s, e);
    const int n_act = __popc(act_lo) + __popc(act_hi);
    if (n_act == 0) {
      if (HETERO && first_chunk)                           // this row contributes nothing: clear its slice
        for (int64_t p = s + lane; p < e; p += 32) dw[p] = 0.f;
      continue;
    }
    if (n_act <= 16) {
      // four 32-synapse stretches per round: their indices first, then for every active batch lane
      // four independent gathers per lane (the kernel is bound by the latency of these L2 gathers)
      constexpr int U = 4;
      for (int64_t pb = s; pb < e; pb += 32 * U) {
        int64_t j[U];
        bool ok[U];
        float acc[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int64_t p = pb + 32 * u + lane;
          ok[u] = p < e;
          j[u] = ok[u] ? (int64_t)__ldg(idx + p) : 0;
          acc[u] = 0.f;
        }
        uint32_t m = act_lo;
        while (m) {                                        // uniform across the warp
          const int src = __ffs(m) - 1;
          m &= m - 1;
          const float a = __shfl_sync(0xffffffffu, a_lo, src);
          const float* __restrict__ crow = ct + (b0 + src) * n_post;
          float c[U];
#pragma unroll
          for (int u = 0; u < U; ++u) c[u] = ok[u] ? __ldg(crow + j[u]) : 0.f;
#pragma unroll
          for (int u = 0; u < U; ++u) acc[u] = fmaf(a, c[u], acc[u]);
        }
        m = act_hi;
        while (m) {
          const int src = __ffs(m) - 1;
          m &= m - 1;
          const float a = __shfl_sync(0xffffffffu, a_hi, src);
          const float* __restrict__ crow = ct + (b0 + 32 + src) * n_post;
          float c[U];
#pragma unroll
          for (int u = 0; u < U; ++u) c[u] = ok[u] ? __ldg(crow + j[u]) : 0.f;
#pragma unroll
          for (int u = 0; u < U; ++u) acc[u] = fmaf(a, c[u], acc[u]);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int64_t p = pb + 32 * u + lane;
          if (ok[u]) {
            if (HETERO) {
              if (first_chunk) dw[p] = acc[u]; else dw[p] += acc[u];
            } else {
              homo_acc += acc[u];
            }
          }
        }
      }
    } else {
      for (int64_t pb = s; pb < e; pb += 32) {
        const int64_t p = pb + lane;
        const int32_t j_l = p < e ? __ldg(idx + p) : 0;
        const int cnt = (int)((e - pb) < 32 ? (e - pb) : 32);
        float dw_l = 0.f;
        for (int t = 0; t < cnt; ++t) {
          const int32_t j = __shfl_sync(0xffffffffu, j_l, t);
          const float* __restrict__ crow = ctT + (int64_t)j * Bp + b0;
          float v = a_lo * __ldg(crow + lane);             // padded batch columns are zero
          if (b0 + 32 < Bp) v = fmaf(a_hi, __ldg(crow + 32 + lane), v);
          v = warp_sum(v);
          if (lane == t) dw_l = v;
        }
        if (p < e) {
          if (HETERO) {
            if (first_chunk) dw[p] = dw_l; else dw[p] += dw_l;
          } else {
            homo_acc += dw_l;
          }
        }
      }
    }
  }
  if (!HETERO) {
    homo_acc = warp_sum(homo_acc);
    if (lane == 0) block_part[threadIdx.x >> 5] = homo_acc;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.f;
      for (int k = 0; k < (int)(blockDim.x >> 5); ++k) t += block_part[k];
      if (t != 0.f) red_add(dw, t);
    }
  }
}

static size_t ctT_bytes(int64_t batch, int64_t n_post) {
  const int64_t Bp = (batch + 31) & ~int64_t(31);
  return ((size_t)n_post * (size_t)Bp * sizeof(float) + 255) & ~size_t(255);
}

}  // namespace bsx

using namespace bsx;

extern "C" {

size_t bsx_vecmat_vjp_batched_workspace_bytes(int64_t batch, int64_t n_post) {
  if (batch < 0 || n_post < 0) return 0;
  return ctT_bytes(batch, n_post);
}

int bsx_vecmat_vjp_batched(const bsx_conn_t* conn, const void* x, int x_format, int event, const float* ct,
                           int64_t batch, float* dx, float* dw, void* workspace, size_t workspace_bytes,
                           bsx_stream_t stream) {
  BSX_TRACE("bsx_vecmat_vjp_batched");
  int rc = check_conn(conn);
  if (rc) return rc;
  if (batch < 0) return fail(BSX_ERR_INVALID_ARG, "negative batch");
  if (x_format != BSX_SPK_BOOL8 && x_format != BSX_SPK_F32)
    return fail(BSX_ERR_INVALID_ARG, "vjp takes the primal input as BOOL8 or F32");
  cudaStream_t st = as_stream(stream);
  const bool empty = conn->n_pre == 0 || (!conn->indptr && conn->conn_num == 0) || conn->n_post == 0;
  if (dw && !conn->hetero) {
    rc = launch_zero(dw, 1, st);
    if (rc) return rc;
  }
  if (batch == 0 || empty) {
    if (dx && batch > 0 && conn->n_pre > 0) return launch_zero(dx, batch * conn->n_pre, st);
    if (dw && conn->hetero && conn->nnz > 0) return launch_zero(dw, conn->nnz, st);
    return BSX_OK;
  }
  if (!ct) return fail(BSX_ERR_INVALID_ARG, "ct is NULL");
  if (dw && !x) return fail(BSX_ERR_INVALID_ARG, "the weight cotangent needs the primal input x");
  if (!dx && !dw) return BSX_OK;
  if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 15) || workspace_bytes < ctT_bytes(batch, conn->n_post))
    return fail(BSX_ERR_WORKSPACE, "batched vjp needs %zu workspace bytes", ctT_bytes(batch, conn->n_post));
  int sms = sm_count();
  if (sms <= 0) return fail(BSX_ERR_CUDA, "no CUDA device");
  const int64_t Bp = (batch + 31) & ~int64_t(31);
  if (Bp / 32 > 65535) return fail(BSX_ERR_UNSUPPORTED, "batch too large");
  float* ctT = static_cast<float*>(workspace);
  rc = launch_transpose_pad(ct, batch, conn->n_post, Bp, ctT, st);
  if (rc) return rc;
  int64_t blocks = (conn->n_pre + 7) / 8;
  if (blocks > (int64_t)sms * 8) blocks = (int64_t)sms * 8;
  if (blocks < 1) blocks = 1;
  const RowMap rm = make_rowmap(conn);
  const bool ev = event != 0;
  for (int64_t b0 = 0; b0 < batch; b0 += 64) {
    const bool first = b0 == 0;
    if (dx) {
      if (conn->hetero)
        vjp_dx_batched_kernel<true><<<(unsigned)blocks, 256, 0, st>>>(rm, conn->indices, conn->weights, ctT, Bp, batch,
                                                                     b0, conn->n_pre, dx);
      else
        vjp_dx_batched_kernel<false><<<(unsigned)blocks, 256, 0, st>>>(rm, conn->indices, conn->weights, ctT, Bp, batch,
                                                                      b0, conn->n_pre, dx);
      BSX_LAUNCH_CHECK("vjp_dx_batched_kernel");
    }
    if (dw) {
#define BSX_VJPW(H, F)                                                                                        \
  vjp_dw_batched_kernel<H, F><<<(unsigned)blocks, 256, 0, st>>>(rm, conn->indices, x, ev, ct, ctT, Bp, batch, b0, \
                                                                conn->n_pre, conn->n_post, dw, first)
      if (conn->hetero) {
        if (x_format == BSX_SPK_BOOL8) BSX_VJPW(true, BSX_SPK_BOOL8); else BSX_VJPW(true, BSX_SPK_F32);
      } else {
        if (x_format == BSX_SPK_BOOL8) BSX_VJPW(false, BSX_SPK_BOOL8); else BSX_VJPW(false, BSX_SPK_F32);
      }
#undef BSX_VJPW
      BSX_LAUNCH_CHECK("vjp_dw_batched_kernel");
    }
  }
  return BSX_OK;
}

}  // extern "C"
