// Launchers shared between the translation units of the bsx library.
#pragma once
#include "common.cuh"

namespace bsx {

// Packs (batch, n) byte/float spikes into (batch, ceil(n/32)) words.
int launch_pack(const void* spikes, int format, int64_t batch, int64_t n, uint32_t* bits, cudaStream_t st);

// Clears hdr, queues the flat positions of all active spikes and, in the same
// launch, zeroes zero_n floats at zero_ptr (may be NULL).
int launch_compact(const void* spikes, int format, int64_t batch, int64_t n_pre, QueueHeader* hdr,
                   uint32_t* entries, float* zero_ptr, int64_t zero_n, cudaStream_t st);

int launch_zero(float* z, int64_t n, cudaStream_t st);

// Shared body of the vecmat entry points (scatter.cu): queue the active rows of
// `in` in the workspace `ws`, then scatter them.  x != NULL multiplies by the value.
int vecmat_common(const bsx_conn_t* conn, const void* in, int format, const float* x, int64_t batch,
                  float* out, int accumulate, void* ws, size_t ws_bytes, int chunk, int blocks_per_sm,
                  cudaStream_t st);

// Batched scatter with the output slice in shared memory (scatter_smem.cu).
bool scatter_smem_applies(const bsx_conn_t* conn, int format, int64_t batch);
bool scatter_smem_preferred(const bsx_conn_t* conn, int format, int64_t batch);
int launch_scatter_smem(const bsx_conn_t* conn, const void* spikes, int format, const float* x, int64_t batch,
                        float* out, int accumulate, cudaStream_t st, int row_mul = 0);   // row_mul >= 1: sliced layout with that many slices

// One-kernel event vecmat for a few spike vectors (scatter_fused.cu): memset node + list-and-scatter kernel.
bool scatter_fused_applies(const bsx_conn_t* conn, const void* spikes, int format, int64_t batch);
bool scatter_fused_fits(const bsx_conn_t* conn, int format, int64_t batch);
int launch_scatter_fused(const bsx_conn_t* conn, const void* spikes, int format, const float* x, int64_t batch,
                         float* out, int accumulate, cudaStream_t st, float* clear_next = nullptr);

// (B, n) row-major -> (n, Bp) row-major, zero padded to Bp (a multiple of 32) columns (vjp_batched.cu).
int launch_transpose_pad(const float* src, int64_t B, int64_t n, int64_t Bp, float* dst, cudaStream_t st);

// Batched event matvec, 16 spike vectors per pass over the indices (gather_batched.cu).
size_t b16_mask_bytes(int64_t batch, int64_t n_post);
bool b16_fits(int64_t n_post);
int launch_event_matvec_b16(const bsx_conn_t* conn, const void* spikes, int format, int64_t batch, float* out,
                            void* workspace, int weight_mode, cudaStream_t st);

}  // namespace bsx
