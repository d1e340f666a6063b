/*
 * Launch-geometry knobs of two bsx kernels, for parameter sweeps and for tests that must
 * reach a particular kernel variant.  Not part of the boundary a binding binds to
 * (include/bsx.h): the symbols are exported by the library, but their meaning may change
 * with the kernels.
 */
#ifndef BSX_TUNING_H_
#define BSX_TUNING_H_

#include "bsx.h"

#ifdef __cplusplus
extern "C" {
#endif

/* bsx_event_vecmat with explicit launch geometry for tuning: entries per work item of a
 * fixed-number row, and resident blocks per SM of the global-atomic kernel.
 * blocks_per_sm = -1 asks for the variant that accumulates output slices of
 * 32768 columns in shared memory wherever it applies (batch >= 16, n_post <=
 * 131072).  With both at 0 (what bsx_event_vecmat passes) the library chooses:
 * the shared-memory variant when batch * slices is at least 3/4 of the SM count
 * and n_post <= 65536, the global-atomic kernel otherwise.  Any positive value
 * keeps the global-atomic kernel. */
int bsx_event_vecmat_tuned(const bsx_conn_t* conn, const void* spikes, int spike_format, int64_t batch,
                           float* out, int accumulate, void* workspace, size_t workspace_bytes,
                           int chunk, int blocks_per_sm, bsx_stream_t stream);

/* bsx_event_matvec with explicit launch geometry for tuning (0 = default).  mask_mode: 1 spike
 * words staged in shared memory by a bulk-async (TMA) copy, 2 staged by ordinary
 * loads, 3 read from global memory, 4 one pass per vector even when batched;
 * batched passes only: 5 stream heterogeneous weights with the indices, 6 fetch
 * them per hit (default: chosen on the device from the spike density).
 * unroll: 128-bit index loads in flight per lane (1, 2, 4 or 6). */
int bsx_event_matvec_tuned(const bsx_conn_t* conn, const void* spikes, int spike_format, int64_t batch,
                           float* out, void* workspace, size_t workspace_bytes, int blocks_per_sm,
                           int mask_mode, int unroll, bsx_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* BSX_TUNING_H_ */
