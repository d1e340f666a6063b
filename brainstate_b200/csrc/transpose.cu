// Construction-time kernels: index validation and the postsynaptic-major
// (transposed) copy of a connectivity, built by a counting sort by column.
//
// The transposed copy lists, for every column j, the stored entries that target
// j in ascending position (= ascending (row, k)) order.  The order inside a
// column is made canonical by a rank sort after the atomic fill, so two builds of
// the same matrix are identical and the gather that walks it sums in a fixed order.
#include "common.cuh"
#include "internal.cuh"

namespace bsx {

__global__ void __launch_bounds__(256)
validate_kernel(RowMap rm, const int32_t* __restrict__ idx, int64_t nnz, int64_t n_pre, int64_t n_post,
                int32_t* __restrict__ status) {
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  bool bad = false;
  for (int64_t p = tid; p < nnz; p += stride) {
    const int32_t j = __ldg(idx + p);
    bad |= (j < 0) || (j >= n_post);
  }
  if (rm.p32 || rm.p64) {
    for (int64_t i = tid; i < n_pre; i += stride) {
      int64_t s, e;
      rm.range(i, s, e);
      bad |= (s < 0) || (e < s) || (e > nnz);
    }
    if (tid == 0) {
      int64_t s, e;
      rm.range(0, s, e);
      bad |= (s != 0);
      rm.range(n_pre - 1, s, e);
      bad |= (e != nnz);
    }
  }
  if (__any_sync(0xffffffffu, bad) && (threadIdx.x & 31) == 0) atomicExch(status, (int32_t)BSX_ERR_INDEX_RANGE);
}

__global__ void __launch_bounds__(256)
hist_kernel(const int32_t* __restrict__ idx, int64_t nnz, int32_t* __restrict__ counts) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t p = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; p < nnz; p += stride)
    atomicAdd(counts + __ldg(idx + p), 1);
}

// Exclusive scan of counts[0..n) by one block; writes int64 offsets (n+1 of them)
// and turns counts into the running cursor (start offset of each column).
__global__ void __launch_bounds__(1024)
scan_kernel(int32_t* __restrict__ counts, int64_t n, int64_t* __restrict__ offsets) {
  __shared__ int64_t warp_tot[32];
  __shared__ int64_t carry_s;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  if (threadIdx.x == 0) carry_s = 0;
  __syncthreads();
  for (int64_t base = 0; base < n; base += 1024) {
    const int64_t i = base + threadIdx.x;
    const int64_t c = (i < n) ? counts[i] : 0;
    int64_t incl = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int64_t t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    if (lane == 31) warp_tot[wid] = incl;
    __syncthreads();
    if (wid == 0) {
      int64_t v = warp_tot[lane];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int64_t t = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += t;
      }
      warp_tot[lane] = v;  // inclusive totals of the warps
    }
    __syncthreads();
    const int64_t carry = carry_s;
    const int64_t excl = carry + (wid ? warp_tot[wid - 1] : 0) + incl - c;
    if (i < n) {
      offsets[i] = excl;
      counts[i] = (int32_t)excl;
    }
    __syncthreads();
    if (threadIdx.x == 1023) carry_s = carry + warp_tot[31];
    __syncthreads();
  }
  if (threadIdx.x == 0) offsets[n] = carry_s;
}

__global__ void __launch_bounds__(256)
fill_kernel_t(const int32_t* __restrict__ idx, int64_t nnz, int32_t* __restrict__ cursor,
              int32_t* __restrict__ tmp_perm) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t p = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; p < nnz; p += stride) {
    const int32_t pos = atomicAdd(cursor + __ldg(idx + p), 1);
    tmp_perm[pos] = (int32_t)p;
  }
}

__device__ __forceinline__ int32_t row_of(const RowMap& rm, int64_t p, int64_t n_pre) {
  if (!rm.p32 && !rm.p64) return (int32_t)(p / rm.K);
  // largest i with start(i) <= p; empty rows share a start, so search on the end offsets
  int64_t lo = 0, hi = n_pre - 1;
  while (lo < hi) {
    const int64_t mid = (lo + hi) >> 1;
    int64_t s, e;
    rm.range(mid, s, e);
    if (e <= p) lo = mid + 1; else hi = mid;
  }
  return (int32_t)lo;
}

// One warp per column: rank sort of the column's entries (all distinct).
__global__ void __launch_bounds__(256)
sort_columns_kernel(RowMap rm, const int64_t* __restrict__ offsets, int64_t n_cols, int64_t n_pre,
                    const int32_t* __restrict__ tmp_perm, int32_t* __restrict__ t_perm,
                    int32_t* __restrict__ t_indices) {
  const int lane = threadIdx.x & 31;
  const int64_t wstep = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t j = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; j < n_cols; j += wstep) {
    const int64_t s = offsets[j], e = offsets[j + 1];
    for (int64_t a = s + lane; a < e; a += 32) {
      const int32_t x = tmp_perm[a];
      int64_t rank = 0;
      for (int64_t t = s; t < e; ++t) rank += (tmp_perm[t] < x);
      t_perm[s + rank] = x;
      t_indices[s + rank] = row_of(rm, x, n_pre);
    }
  }
}

__global__ void __launch_bounds__(256)
permute_kernel(const float* __restrict__ src, const int32_t* __restrict__ perm, int64_t n,
               float* __restrict__ dst) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t p = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; p < n; p += stride)
    dst[p] = __ldg(src + __ldg(perm + p));
}

static unsigned flat_grid(int64_t n, int sms) {
  int64_t blocks = (n + 255) / 256;
  if (blocks < 1) blocks = 1;
  if (blocks > (int64_t)sms * 16) blocks = (int64_t)sms * 16;
  return (unsigned)blocks;
}

static size_t align256(size_t b) { return (b + 255) & ~size_t(255); }

}  // namespace bsx

using namespace bsx;

extern "C" {

int bsx_validate_conn(const bsx_conn_t* conn, int32_t* status_word, bsx_stream_t stream) {
  BSX_TRACE("bsx_validate_conn");
  int rc = check_conn(conn);
  if (rc) return rc;
  if (!status_word) return fail(BSX_ERR_INVALID_ARG, "status word is NULL");
  if (conn->nnz == 0 && !conn->indptr) return BSX_OK;
  if (conn->n_pre == 0) return BSX_OK;
  int sms = sm_count();
  if (sms <= 0) return fail(BSX_ERR_CUDA, "no CUDA device");
  int64_t work = conn->nnz > conn->n_pre ? conn->nnz : conn->n_pre;
  validate_kernel<<<flat_grid(work, sms), 256, 0, as_stream(stream)>>>(
      make_rowmap(conn), conn->indices, conn->nnz, conn->n_pre, conn->n_post, status_word);
  BSX_LAUNCH_CHECK("validate_kernel");
  return BSX_OK;
}

size_t bsx_transpose_workspace_bytes(int64_t n_pre, int64_t n_post, int64_t nnz) {
  (void)n_pre;
  if (n_post < 0 || nnz < 0) return 0;
  return align256(sizeof(int32_t) * (size_t)(n_post + 1)) + align256(sizeof(int32_t) * (size_t)nnz);
}

int bsx_transpose_build(const bsx_conn_t* conn, int64_t nnz, int64_t* t_indptr, int32_t* t_indices,
                        int32_t* t_perm, void* workspace, size_t workspace_bytes, bsx_stream_t stream) {
  BSX_TRACE("bsx_transpose_build");
  int rc = check_conn(conn);
  if (rc) return rc;
  if (nnz != conn->nnz) return fail(BSX_ERR_INVALID_ARG, "nnz argument differs from conn->nnz");
  if (nnz >= (int64_t)INT32_MAX) return fail(BSX_ERR_UNSUPPORTED, "transpose needs nnz < 2^31");
  if (!t_indptr) return fail(BSX_ERR_INVALID_ARG, "t_indptr is NULL");
  if (nnz > 0 && (!t_indices || !t_perm)) return fail(BSX_ERR_INVALID_ARG, "transposed arrays are NULL");
  if (!workspace || workspace_bytes < bsx_transpose_workspace_bytes(conn->n_pre, conn->n_post, nnz))
    return fail(BSX_ERR_WORKSPACE, "transpose needs %zu workspace bytes",
                bsx_transpose_workspace_bytes(conn->n_pre, conn->n_post, nnz));
  int sms = sm_count();
  if (sms <= 0) return fail(BSX_ERR_CUDA, "no CUDA device");
  cudaStream_t st = as_stream(stream);
  int32_t* counts = static_cast<int32_t*>(workspace);
  int32_t* tmp_perm = reinterpret_cast<int32_t*>(static_cast<char*>(workspace) +
                                                 align256(sizeof(int32_t) * (size_t)(conn->n_post + 1)));
  BSX_CUDA(cudaMemsetAsync(counts, 0, sizeof(int32_t) * (size_t)(conn->n_post + 1), st));
  if (nnz > 0) {
    hist_kernel<<<flat_grid(nnz, sms), 256, 0, st>>>(conn->indices, nnz, counts);
    BSX_LAUNCH_CHECK("hist_kernel");
  }
  scan_kernel<<<1, 1024, 0, st>>>(counts, conn->n_post, t_indptr);
  BSX_LAUNCH_CHECK("scan_kernel");
  if (nnz > 0) {
    fill_kernel_t<<<flat_grid(nnz, sms), 256, 0, st>>>(conn->indices, nnz, counts, tmp_perm);
    BSX_LAUNCH_CHECK("fill_kernel_t");
    int64_t blocks = (conn->n_post + 7) / 8;
    if (blocks > (int64_t)sms * 8) blocks = (int64_t)sms * 8;
    if (blocks < 1) blocks = 1;
    sort_columns_kernel<<<(unsigned)blocks, 256, 0, st>>>(make_rowmap(conn), t_indptr, conn->n_post,
                                                          conn->n_pre, tmp_perm, t_perm, t_indices);
    BSX_LAUNCH_CHECK("sort_columns_kernel");
  }
  return BSX_OK;
}

int bsx_permute_f32(const float* src, const int32_t* perm, int64_t n, float* dst, bsx_stream_t stream) {
  if (n < 0) return fail(BSX_ERR_INVALID_ARG, "negative length");
  if (n == 0) return BSX_OK;
  if (!src || !perm || !dst) return fail(BSX_ERR_INVALID_ARG, "bsx_permute_f32: NULL buffer");
  int sms = sm_count();
  if (sms <= 0) return fail(BSX_ERR_CUDA, "no CUDA device");
  permute_kernel<<<flat_grid(n, sms), 256, 0, as_stream(stream)>>>(src, perm, n, dst);
  BSX_LAUNCH_CHECK("permute_kernel");
  return BSX_OK;
}

}  // extern "C"
