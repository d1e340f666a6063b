/*
 * bsx — event-driven synaptic propagation on NVIDIA B200 (sm_100a), C ABI.
 *
 * This is the boundary a binding of brainstate's event-connection layers binds
 * to.  In the reference, brainstate/nn/_event_fixedprob.py builds the
 * connectivity and hands every product to the third-party package brainevent
 * (`x @ brainevent.FixedPostNumConn(...)`, `x @ brainevent.CSR(...)`); each entry
 * point below replaces one of those dispatches, cited beside it by the
 * reference file:line that reaches it.
 *
 * Conventions
 *  - Every pointer is a DEVICE pointer unless its name starts with `host_`.
 *    The caller owns every buffer, workspace included; nothing here allocates
 *    (the bsx_ipc_* set-up helpers and the host generator handle excepted).
 *  - All work is enqueued on the caller's stream (a cudaStream_t passed as
 *    void*); functions return as soon as the work is enqueued.
 *  - Return value: BSX_OK or a negative bsx_status_t.  Nothing is thrown across
 *    the boundary; bsx_last_error_string() describes the calling thread's last
 *    failure.  Kernel-side checks (index range, queue overflow) are reported
 *    through a caller-provided device status word, read with bsx_read_status().
 *  - There is no CPU implementation behind these symbols.  Without a CUDA
 *    device every compute entry point returns BSX_ERR_CUDA.
 *  - Re-entrant: the only mutable global state is the thread-local error string and
 *    the built-in queue of bsx_event_vecmat_static (documented there).
 */
#ifndef BSX_H_
#define BSX_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BSX_VERSION 100

typedef void* bsx_stream_t; /* cudaStream_t */

typedef enum {
  BSX_OK = 0,
  BSX_ERR_INVALID_ARG = -1, /* null pointer, negative size, inconsistent layout */
  BSX_ERR_CUDA = -2,        /* a CUDA runtime call failed (no device, launch error) */
  BSX_ERR_INDEX_RANGE = -3, /* a connectivity index lies outside [0, n_post) */
  BSX_ERR_WORKSPACE = -4,   /* workspace pointer null, misaligned or too small */
  BSX_ERR_UNSUPPORTED = -5, /* a size beyond what the kernels address */
  BSX_ERR_TIMEOUT = -6,     /* a bounded device-side wait ran out */
  BSX_ERR_NONFINITE = -7    /* a neuron's potential or synaptic variable became NaN or infinite (network step) */
} bsx_status_t;

/* How a spike vector is stored. */
typedef enum {
  BSX_SPK_BOOL8 = 0,  /* one byte per neuron, nonzero = spike (jax bool) */
  BSX_SPK_F32 = 1,    /* float32, nonzero = unit event (brainevent.EventArray of a float array,
                         brainstate/nn/_event_linear.py:82-85) */
  BSX_SPK_BITS32 = 2, /* packed: bit (i % 32) of uint32 word (i / 32); rows padded to whole words */
  BSX_SPK_LIST = 3    /* compacted active indices: int32 count at list[0], then the indices */
} bsx_spike_format_t;

/*
 * Sparse connectivity with out-degree layout, the data of
 * brainevent.FixedPostNumConn((weight, indices), shape=(n_pre, n_post))
 * (brainstate/nn/_event_fixedprob.py:176-181) when indptr == NULL, and of
 * brainevent.CSR((weight, indices, indptr), shape=...) (:191-196) otherwise.
 */
typedef struct bsx_conn {
  int64_t n_pre;          /* rows */
  int64_t n_post;         /* columns */
  int64_t conn_num;       /* K: entries per row when indptr == NULL */
  int64_t nnz;            /* stored entries: n_pre*K, or indptr[n_pre] */
  const int32_t* indices; /* (n_pre*K) row-major, or (nnz) */
  const void* indptr;     /* NULL, or (n_pre+1) row offsets */
  int32_t indptr_is_64;   /* 0: int32 offsets (the reference's dtype), 1: int64 */
  int32_t hetero;         /* 0: weights points at ONE float; 1: one float per index */
  const float* weights;
} bsx_conn_t;

/* ---- diagnostics ------------------------------------------------------- */
int bsx_version(void);
const char* bsx_last_error_string(void);
const char* bsx_status_name(int status);
/* Number of CUDA devices visible, or 0 (never fails). */
int bsx_device_count(void);
/* Copies the device status word to *host_status after synchronising `stream`.
 * The word is 0 or a bsx_status_t written by a kernel. */
int bsx_read_status(const int32_t* status_word, int32_t* host_status, bsx_stream_t stream);

/* ---- connectivity generation (host) ------------------------------------ */
/*
 * Replaces `rng.randint(0, n_post, size=(n_pre, conn_num))` + the int32 cast of
 * brainstate/nn/_event_fixedprob.py:165-171, bit for bit (MT19937, masked
 * rejection), without the int64 intermediate.  Rows [row_begin, row_end) of the
 * matrix are written to host_out; entries of the other rows are drawn and
 * dropped, so every rank of a sharded job can replay the one stream.
 * If col_begin < col_end only targets inside [col_begin, col_end) are kept
 * (stored minus col_begin) and host_row_counts[row - row_begin] receives how
 * many each row kept (a CSR block for one postsynaptic shard); host_out then
 * needs room for (row_end-row_begin)*conn_num entries in the worst case.
 * Returns the number of entries written, or a negative status.
 */
int64_t bsx_host_fixed_num_indices(uint32_t seed, int64_t n_pre, int64_t n_post, int64_t conn_num,
                                   int64_t row_begin, int64_t row_end,
                                   int64_t col_begin, int64_t col_end,
                                   int32_t* host_out, int32_t* host_row_counts);

/* The same stream in stateful form, for matrices drawn in row chunks (a 32 GB index
 * matrix is produced and uploaded piece by piece): create, draw the next `rows` rows,
 * free.  With a column window only targets inside it are kept; host_k_out (may be
 * NULL) receives the position k of every kept entry inside its row, host_row_counts
 * (may be NULL) how many each row kept.  conn_num < 32768. */
void* bsx_host_gen_new(uint32_t seed);
void bsx_host_gen_free(void* gen);
int64_t bsx_host_gen_rows(void* gen, int64_t rows, int64_t n_post, int64_t conn_num, int64_t col_begin,
                          int64_t col_end, int32_t* host_out, int16_t* host_k_out, int32_t* host_row_counts);

/* Rows of conn_num distinct targets (sampling without replacement) from the same
 * generator; the library's sampler for allow_multi_conn=False
 * (brainstate/nn/_event_fixedprob.py:39-62).  Honours that function's contract but not
 * its numbers, which the reference draws from JAX's threefry generator. */
int64_t bsx_host_distinct_indices(uint32_t seed, int64_t n_pre, int64_t n_post, int64_t conn_num,
                                  int32_t* host_out);

/*
 * Heterogeneous weights keyed by position: w(row, k) = sign * exp(mu + sigma * z), z a
 * standard normal derived from a hash of (seed, row0 + row, k).  kpos (may be NULL: k is
 * the offset inside the row) gives k for every stored entry, as bsx_host_gen_rows
 * reports it for a column-filtered block.  Stands for a `conn_weight` initializer
 * callable (brainstate/nn/_event_fixedprob.py:173-175) at sizes where the weights are
 * generated on the device; bsx_lognormal_weight_at is the same value on the host.
 */
int bsx_lognormal_weights(const bsx_conn_t* conn, const int16_t* kpos, int64_t row0, uint32_t seed, double mu,
                          double sigma, float sign, float* weights_out, bsx_stream_t stream);
float bsx_lognormal_weight_at(uint32_t seed, uint32_t row, uint32_t k, double mu, double sigma, float sign);

/* ---- construction-time checks and derived layouts ---------------------- */
/* Writes BSX_ERR_INDEX_RANGE to *status_word if any index is outside [0, n_post)
 * or indptr is not non-decreasing; leaves it untouched otherwise.  The reference
 * performs no such check (a malformed layout aborts inside brainevent,
 * brainstate/nn/_event_fixedprob.py:124-134). */
int bsx_validate_conn(const bsx_conn_t* conn, int32_t* status_word, bsx_stream_t stream);

/* Spike packing: any format except LIST -> BITS32 words ((n+31)/32 per batch row). */
int bsx_pack_spikes(const void* spikes, int spike_format, int64_t batch, int64_t n,
                    uint32_t* bits, bsx_stream_t stream);

/*
 * Transposed (postsynaptic-major) copy of a connectivity: for every column j the
 * source rows that target it, in ascending (row, k) order.
 *   t_indptr  (n_post+1) int64   row offsets of the transposed matrix
 *   t_indices (nnz)      int32   presynaptic row of each entry
 *   t_perm    (nnz)      int32   position of the entry in the original arrays
 *                                (gathers weights after `with_data`,
 *                                 brainstate/nn/_event_fixedprob.py:204)
 * Requires nnz < 2^31.  The transposed matrix, read as a bsx_conn_t with
 * n_pre/n_post swapped, turns bsx_event_matvec into the deterministic
 * post-centric form of the forward product.
 */
size_t bsx_transpose_workspace_bytes(int64_t n_pre, int64_t n_post, int64_t nnz);
int bsx_transpose_build(const bsx_conn_t* conn, int64_t nnz, int64_t* t_indptr, int32_t* t_indices,
                        int32_t* t_perm, void* workspace, size_t workspace_bytes,
                        bsx_stream_t stream);
/* dst[p] = src[perm[p]] — weights of the transposed copy. */
int bsx_permute_f32(const float* src, const int32_t* perm, int64_t n, float* dst, bsx_stream_t stream);

/* ---- forward products -------------------------------------------------- */
/*
 * y = EventArray(spk) @ conn            brainstate/nn/_event_fixedprob.py:249-252 -> :204-205
 *   y[b, idx[i,k]] += w[i,k]  for every i with spk[b,i] != 0   (pre-centric scatter)
 * spikes: (batch, n_pre) in `spike_format`; out: (batch, n_post) float32.
 * accumulate == 0 zeroes `out` first.  Workspace: bsx_event_vecmat_workspace_bytes.
 * Spike inputs of up to 128 KB (one bool vector of 131 072 neurons) in a 16-byte aligned
 * buffer run as a memset node plus ONE kernel (active-row list in shared memory + scatter),
 * which leaves the workspace untouched.
 * Duplicate targets accumulate (brainstate/nn/_event_fixedprob_test.py:256-259).
 * Summation order of heterogeneous weights is not fixed between runs (atomic adds).
 */
size_t bsx_event_vecmat_workspace_bytes(int64_t batch, int64_t n_pre);
int bsx_event_vecmat(const bsx_conn_t* conn, const void* spikes, int spike_format, int64_t batch,
                     float* out, int accumulate, void* workspace, size_t workspace_bytes,
                     bsx_stream_t stream);
/* Which kernel bsx_event_vecmat runs for this connectivity, spike format and batch:
 * BSX_VECMAT_GLOBAL_ATOMICS (compaction launch + scatter launch, uses the workspace) or
 * BSX_VECMAT_SHARED_SLICES (one launch, workspace untouched).  Negative on invalid input. */
#define BSX_VECMAT_GLOBAL_ATOMICS 0
#define BSX_VECMAT_SHARED_SLICES 1
int bsx_event_vecmat_variant(const bsx_conn_t* conn, int spike_format, int64_t batch);
/* Kernel launches one bsx_event_vecmat call of this shape enqueues (a diagnostic for
 * callers that budget launch latency, e.g. one spike vector per simulation step). */
int bsx_event_vecmat_launches(const bsx_conn_t* conn, int spike_format, int64_t batch);

/*
 * Sliced layout for the shared-memory variant.  No counterpart in the reference: a
 * derived copy, like the transposed one.  The entries of every row are grouped by
 * output slice (slice = column / 32768), so that the block that owns a slice reads
 * only its own entries instead of the whole row; inside a group they are sorted by
 * column mod 32 (original order kept among equals) and dealt round-robin over the
 * group's 32-entry stretches, so that the 32 entries a warp adds to shared memory
 * in one instruction fall into distinct banks as far as the group allows:
 *   s_indptr  (n_pre*S+1) int64   start of group (row, slice) = entry row*S + slice;
 *                                 S = bsx_sliced_slices(n_post), at most 4
 *   s_indices (nnz)       int32   the targets, regrouped
 *   s_perm    (nnz)       int32   position of each entry in the original arrays
 *                                 (weights of the copy = bsx_permute_f32(w, s_perm))
 * With s_indices = s_perm = NULL only s_indptr is written (rows that are already
 * grouped, e.g. sorted targets, can then be scattered from the original arrays; they
 * give the right sums but not the bank-friendly order).
 * bsx_event_vecmat_sliced takes a bsx_conn_t whose indptr is s_indptr (64-bit), whose
 * indices/weights are the regrouped arrays and whose n_pre, n_post, nnz, hetero are
 * those of the original, and computes what bsx_event_vecmat computes, in one launch
 * with no workspace.  It is worth calling where bsx_event_vecmat_variant answers
 * BSX_VECMAT_SHARED_SLICES; below that batch size it leaves SMs idle.
 */
int64_t bsx_sliced_slices(int64_t n_post);
int bsx_sliced_build(const bsx_conn_t* conn, int64_t* s_indptr, int32_t* s_indices, int32_t* s_perm,
                     bsx_stream_t stream);
int bsx_event_vecmat_sliced(const bsx_conn_t* sliced, const void* spikes, int spike_format, int64_t batch,
                            float* out, int accumulate, bsx_stream_t stream);

/*
 * Deterministic form of the sliced scatter.  No counterpart in the reference.  Heterogeneous
 * weights are summed in 2^-scale_log2 fixed point (signed 32-bit, native shared-memory integer
 * atomics), so the result does not depend on the order in which the GPU adds: identical on
 * every run, and a drop-in for the order-fixing gather at the speed of the scatter.  The
 * price is absolute precision: every addend is rounded to 2^-scale_log2, so an output is
 * within (number of its events) * 2^-(scale_log2+1) of the exact sum.  bsx_fixed_scale_log2
 * picks the largest scale that cannot overflow: it sums |w| per output column (order-free
 * itself), takes the largest column B and returns floor(log2(2^30 / B)) in *host_scale_log2
 * (it synchronises the stream; call it once per weight array, not per product).  For the
 * 65 536 x 655 matrix with weights ~ N(0.1, 0.01), B = 73 and the scale is 2^-23: an output of
 * 7 events is within 4e-7 of the exact sum.  Homogeneous weights need no scale (events are
 * counted); the sliced entry point is then called as it is.
 */
size_t bsx_fixed_scale_workspace_bytes(int64_t n_post);
int bsx_fixed_scale_log2(const bsx_conn_t* conn, void* workspace, size_t workspace_bytes, int32_t* host_scale_log2,
                         bsx_stream_t stream);
int bsx_event_vecmat_sliced_fixed(const bsx_conn_t* sliced, const void* spikes, int spike_format, int64_t batch,
                                  float* out, int accumulate, int32_t scale_log2, bsx_stream_t stream);

/*
 * The per-step call of a simulation loop without its clearing node.  No counterpart in the
 * reference.  For spike inputs of up to 128 KB (16-byte aligned) bsx_event_vecmat runs a memset
 * node and one kernel; a loop that alternates between two output buffers can fold the clearing
 * into the kernel: bsx_event_vecmat_chained ADDS the product to `out` (which the previous call of
 * the chain, or the caller before the first one, has cleared) and clears `next_out` (batch * n_post
 * floats, another buffer than `out`; NULL: nothing is cleared) for the call that follows — one
 * launch per call, no workspace.  Larger inputs answer BSX_ERR_UNSUPPORTED.
 */
int bsx_event_vecmat_chained(const bsx_conn_t* conn, const void* spikes, int spike_format, int64_t batch,
                             float* out, float* next_out, bsx_stream_t stream);

/*
 * Compressed form of the sliced layout (index compression; no counterpart in the reference).
 * Inside a group every column lies in one 32 768-column slice, so 16 bits hold it:
 * bsx_sliced_compress writes local[p] = indices[p] - 32768 * slice (0xffff for a column outside
 * the matrix) for the regrouped indices of `sliced`; bsx_quantize_f32 writes
 * q[p] = round_to_nearest_even(w[p] * 2^scale_log2), the addend bsx_event_vecmat_sliced_fixed
 * forms per event.  bsx_event_vecmat_sliced16 is the scatter over them: `sliced` gives the group
 * offsets, sizes and, for homogeneous weights, the weight; its indices are not read.  Results are
 * bit-identical to bsx_event_vecmat_sliced_fixed (heterogeneous; qweights must come from the same
 * scale_log2) and to bsx_event_vecmat_sliced (homogeneous; qweights NULL, scale_log2 ignored) while
 * the kernel reads 6 instead of 8 bytes per synapse (2 instead of 4) and does no arithmetic per
 * event besides the add.
 */
int bsx_sliced_compress(const bsx_conn_t* sliced, uint16_t* local, bsx_stream_t stream);
int bsx_quantize_f32(const float* w, int64_t n, int32_t scale_log2, int32_t* q, bsx_stream_t stream);
int bsx_event_vecmat_sliced16(const bsx_conn_t* sliced, const uint16_t* local, const int32_t* qweights,
                              const void* spikes, int spike_format, int64_t batch, float* out, int accumulate,
                              int32_t scale_log2, bsx_stream_t stream);

/*
 * Event vecmat without a workspace argument.  No counterpart in the reference:
 * it exists for callers that cannot obtain device memory when they call (a
 * custom-call handler inside a framework that owns the GPU's memory pool; a
 * latency-critical loop that must avoid the device-wide stall of an allocation).
 * Same result as bsx_event_vecmat.  The active-row queue lives in a 4 MiB array
 * built into the library image (each GPU that loads the library holds it until
 * the process exits), which limits the input to
 *     batch * n_pre <= BSX_STATIC_QUEUE_MAX_SPIKES
 * (BSX_SPK_LIST inputs need no queue and are not limited); larger inputs are
 * refused with BSX_ERR_WORKSPACE.  The call allocates nothing.  Its first call on
 * a device looks up the array's device address (cudaGetSymbolAddress, with that
 * device current), so make that first call outside any stream capture.  All calls
 * on one GPU share the one array: calls that may run concurrently on the device
 * (different streams) race on it and must be serialised by the caller.
 */
#define BSX_STATIC_QUEUE_MAX_SPIKES 1048000
int bsx_event_vecmat_static(const bsx_conn_t* conn, const void* spikes, int spike_format, int64_t batch,
                            float* out, int accumulate, bsx_stream_t stream);

/*
 * y = x @ conn for float x               brainstate/nn/_event_fixedprob.py:202-205
 *   y[b, idx[i,k]] += x[b,i] * w[i,k]   (rows with x == 0 are skipped)
 * Also the two terms of the forward-mode rule (_event_fixedprob_test.py:90-126).
 */
int bsx_float_vecmat(const bsx_conn_t* conn, const float* x, int64_t batch, float* out,
                     int accumulate, void* workspace, size_t workspace_bytes, bsx_stream_t stream);

/*
 * y = conn @ EventArray(s): y[b,i] = sum_k w[i,k] * [s[b, idx[i,k]] != 0]
 * (the "W @ spike" product; deterministic gather, one warp per row, spike
 * bitmask staged in shared memory).  spikes: (batch, n_post); out: (batch, n_pre).
 * With batch >= 2 and a workspace of bsx_event_matvec_workspace_bytes, one pass
 * over the indices serves 16 spike vectors at a time; otherwise each vector is a
 * pass of its own (the workspace then only holds packed spike words, and may be
 * NULL for BITS32 input).
 */
size_t bsx_event_matvec_workspace_bytes(int64_t batch, int64_t n_post);
int bsx_event_matvec(const bsx_conn_t* conn, const void* spikes, int spike_format, int64_t batch,
                     float* out, void* workspace, size_t workspace_bytes, bsx_stream_t stream);
/*
 * y = conn @ v for float v: y[b,i] = sum_k w[i,k] * v[b, idx[i,k]].
 * This is the input cotangent of the vecmat (transpose product used by jax.grad,
 * brainstate/nn/_event_fixedprob_test.py:56-88).
 */
int bsx_float_matvec(const bsx_conn_t* conn, const float* v, int64_t batch, float* out,
                     bsx_stream_t stream);

/*
 * y = EventArray(spk) @ W for a dense row-major W (n_pre, n_post)
 *                                          brainstate/nn/_event_linear.py:99-100
 *   y[b, :] = sum over i with spk[b,i] != 0 of W[i, :]   (ascending i, no atomics)
 */
int bsx_dense_event_vecmat(const void* spikes, int spike_format, const float* weight, int64_t batch,
                           int64_t n_pre, int64_t n_post, float* out, bsx_stream_t stream);

/*
 * Weight cotangent of the dense event product:      brainstate/nn/_event_linear.py:99-100,
 *   dW[i, :] = sum over b with spk[b,i] != 0 of ct[b, :]        tests _event_linear_test.py:51-124
 * (ascending b, no atomics).  dW (n_pre, n_post) is overwritten; n_pre <= 65535 per call.
 * The input cotangent of that product, ct @ W^T, is a plain dense GEMM and is left to a GEMM library.
 */
int bsx_dense_event_dw(const void* spikes, int spike_format, const float* ct, int64_t batch, int64_t n_pre,
                       int64_t n_post, float* dw, bsx_stream_t stream);
/*
 * Scalar-weight form of the dense event layer       brainstate/nn/_event_linear.py:77-97
 *   y[b, :] = r[b] * w,  r[b] = count(spk[b, :] != 0) (float_as_event) or sum(spk[b, :])
 * weight points at ONE float; reduced (may be NULL) receives r (batch).
 */
int bsx_dense_event_scalar(const void* spikes, int spike_format, const float* weight, int float_as_event,
                           int64_t batch, int64_t n_pre, int64_t n_post, float* out, float* reduced,
                           bsx_stream_t stream);

/* ---- reverse-mode products --------------------------------------------- */
/*
 * Cotangents of y = x @ conn for output cotangent ct (batch, n_post), one pass
 * over the indices (brainstate/nn/_event_fixedprob_test.py:56-88):
 *   dx[b,i]  = sum_k w[i,k] ct[b, idx[i,k]]                     (dx may be NULL)
 *   hetero:  dw[i,k] = sum_b a[b,i] ct[b, idx[i,k]]             (dw may be NULL)
 *   homo:    dw[0]   = sum_b sum_i a[b,i] sum_k ct[b, idx[i,k]]
 * a = x (x_format == BSX_SPK_F32 and event == 0) or the event indicator [x != 0].
 * dw is overwritten.  x: (batch, n_pre) in x_format (BOOL8 or F32).
 */
int bsx_vecmat_vjp(const bsx_conn_t* conn, const void* x, int x_format, int event,
                   const float* ct, int64_t batch, float* dx, float* dw, bsx_stream_t stream);

/*
 * The same cotangents for a batch (the training step of the batched event matmul):
 * ct is transposed once into the workspace so that each index serves 64 batch lanes
 * with two coalesced loads; dw only visits the batch lanes where the row fired.
 * Deterministic (no atomics) for heterogeneous weights.
 */
size_t bsx_vecmat_vjp_batched_workspace_bytes(int64_t batch, int64_t n_post);
int bsx_vecmat_vjp_batched(const bsx_conn_t* conn, const void* x, int x_format, int event, const float* ct,
                           int64_t batch, float* dx, float* dw, void* workspace, size_t workspace_bytes,
                           bsx_stream_t stream);

/* ---- fused E/I network step ------------------------------------------------ */
/*
 * Constants of the leaky integrate-and-fire neurons and exponential synapses of
 * an excitatory/inhibitory network.  The host computes the exponentials in double
 * and rounds once, so host and device use the same float32 factors.
 */
typedef struct bsx_lif_params {
  float dt;          /* step */
  float decay_e;     /* exp(-dt/tau_e) */
  float decay_i;     /* exp(-dt/tau_i) */
  float inv_tau_m;   /* 1/tau_m */
  float cuba_gain;   /* 1 - exp(-dt/tau_m) */
  float V_rest, V_th, V_reset;
  float R, I_ext;    /* membrane resistance, constant external current */
  float E_e, E_i;    /* reversal potentials (conductance-based only) */
  int32_t ref_steps; /* refractory period in steps */
  int32_t coba;      /* 0: current-based (CUBA), 1: conductance-based (COBA) */
  /* Background drive: at every step each neuron receives one external excitatory
   * event of size ext_weight when bsx_drive_hash(ext_seed, neuron, step) <
   * ext_threshold (probability ext_threshold / 2^32 per step; 0 switches it off). */
  uint32_t ext_threshold;
  uint32_t ext_seed;
  float ext_weight;
} bsx_lif_params_t;

/*
 * One rank's part of an E/I network.  Global neuron ids [0, n_exc) are excitatory,
 * [n_exc, n_global) inhibitory.  The rank owns neurons [first, first + n_local)
 * (first a multiple of 32) and, of both projections, the synapses that TARGET
 * them: `exc` has n_exc rows, `inh` has n_global - n_exc rows, both have n_local
 * columns (local ids).  On one GPU first = 0 and n_local = n_global.
 */
typedef struct bsx_net {
  int64_t n_global, n_exc, first, n_local;
  bsx_conn_t exc, inh;
  float* V;            /* (n_local) membrane potential */
  float* g_e;          /* (n_local) excitatory synaptic variable */
  float* g_i;          /* (n_local) inhibitory synaptic variable */
  int32_t* ref;        /* (n_local) remaining refractory steps */
  float* delta_e;      /* (n_local) scatter target, zero between steps */
  float* delta_i;      /* (n_local) */
  uint32_t* bits;      /* (ceil(n_global/32)) packed spikes of the latest step, whole network */
  int32_t* lists;      /* ring of `ring` spike lists of n_global + 1 ints each: [count, global ids...];
                          the spikes of step t live in list t % ring; zero the counts before step 0 */
  int32_t ring;        /* >= max(delay_e, delay_i) + 2 */
  int32_t delay_e;     /* steps an excitatory spike waits beyond the next step (synaptic delay) */
  int32_t delay_i;     /* same for inhibitory spikes */
} bsx_net_t;

/*
 * Runs steps [step0, step0 + steps) of a whole network on one GPU in ONE cooperative
 * launch.  This fuses what the reference's examples run as separate operators per
 * step (examples/400_CUBA_2005_bpu.py:60-66: two EventFixedProb products, two Expon
 * updates, CUBA/COBA output, LIFRef update).  Step t consumes the excitatory spikes
 * of step t-1-delay_e and the inhibitory spikes of step t-1-delay_i (the bit-packed
 * counterpart of the reference's delay ring buffer, brainstate/nn/_delay.py:768-958)
 * and leaves its own spikes in list t % ring and in `bits`.
 * raster (may be NULL): (steps, ceil(n/32)) packed spike words; spike_counts (may
 * be NULL): spikes per step.  blocks: grid size, 0 = chosen from the network size.
 */
int bsx_net_run(const bsx_net_t* net, const bsx_lif_params_t* params, int32_t steps, int64_t step0,
                uint32_t* raster, int32_t* spike_counts, int32_t blocks, bsx_stream_t stream);
/* The pieces of step `step`, for the multi-GPU driver: scatter (the delayed spikes
 * of all ranks onto this rank's neurons) -> update (writes the rank's words of
 * `bits`, adds its spike count to *local_count, which may be NULL) -> exchange of
 * the spike words by the caller -> list (fills list step % ring from `bits`). */
int bsx_net_scatter(const bsx_net_t* net, int64_t step, bsx_stream_t stream);
int bsx_net_update(const bsx_net_t* net, const bsx_lif_params_t* params, int64_t step, int32_t* local_count,
                   bsx_stream_t stream);
int bsx_net_list_from_bits(const bsx_net_t* net, int64_t step, bsx_stream_t stream);
/* The same pieces for a driver that overlaps the exchange with the scatter of the rank's own
 * spikes.  bsx_net_list_from_bits_part with rest == 0 empties list step % ring, lists the words
 * [word0, word1) of `bits` (the rank's own words, valid before the exchange) and stores the list's
 * length in marks[step % ring] (device memory, `ring` entries); with rest != 0 it appends all words
 * outside [word0, word1) (after the exchange).  bsx_net_scatter_part scatters, of every list that
 * bsx_net_scatter(step) would read, the entries before its mark (rest == 0) or from its mark on
 * (rest != 0); the two calls together equal bsx_net_scatter(step). */
int bsx_net_list_from_bits_part(const bsx_net_t* net, int64_t step, int64_t word0, int64_t word1, int32_t rest,
                                int32_t* marks, bsx_stream_t stream);
int bsx_net_scatter_part(const bsx_net_t* net, int64_t step, const int32_t* marks, int32_t rest, bsx_stream_t stream);
/*
 * One rank's shard of an E/I network for bsx_net_run_sharded.  Neurons and projections
 * as in bsx_net_t (the rank owns neurons [first, first + n_local) and the synapses that
 * target them; on one GPU first = 0 and n_local = n_global).  The pending synaptic input
 * is kept as a ring of increment rows instead of a ring of spike lists:
 *   incr_e, incr_i  (ring, n_local); row (s % ring) holds what step s will add to g_e /
 *                   g_i and is cleared by that step.  A spike of step s from a projection
 *                   with delay d lands in row (s + 1 + d) % ring.  This is the delay ring
 *                   buffer of brainstate/nn/_delay.py:768-958 applied to the summed
 *                   synaptic input.  Zero before step 0; part of the state afterwards.
 *   fixed_point     0: float32 rows, atomic float adds (the last bit of a heterogeneous
 *                   sum depends on the arrival order).  1: int64 rows holding
 *                   round(w * 2^32) sums — integer addition is associative, so currents
 *                   and rasters are identical for any grid, arrival order and number of
 *                   GPUs; needs |sum of weights per neuron and step| < 2^31.
 *   bits            (ceil(n_local/32)) the rank's spike words of the launch's last step; may be NULL
 */
typedef struct bsx_net_shard {
  int64_t n_global, n_exc, first, n_local;
  bsx_conn_t exc, inh;
  float* V;
  float* g_e;
  float* g_i;
  int32_t* ref;
  void* incr_e;
  void* incr_i;
  uint32_t* bits;
  int32_t ring;        /* >= max(delay_e, delay_i) + 2 */
  int32_t delay_e;
  int32_t delay_i;
  int32_t fixed_point;
} bsx_net_shard_t;

/*
 * How the ranks of one node reach each other.  No counterpart in the reference, which
 * runs on one device.  Every rank launches the same grid (bsx_net_shard_geometry, from
 * words_per_rank): block b of rank r owns spike words [b * words_per_block, ...) of the
 * rank.  After its update, block b pushes the ids of its neurons that spiked into every
 * peer's inbox with plain 64-bit stores over NVLink (peer memory mapped by CUDA IPC);
 * each word is (tag << 32 | payload) with tag = low 32 bits of (exchange sequence number
 * + 1), the first word of a list carrying the count, so a reader knows a word is current
 * by its tag alone: no fence, no separate flag, no collective call and no host round
 * trip per step.
 *   inbox[r]   rank r's inbox as addressable from THIS rank (inbox[rank] is local):
 *              bsx_net_inbox_bytes() bytes, zero at set-up, laid out
 *              [slot][source rank][source block][1 + 32 * words_per_block] uint64
 *   slots      inbox ring depth, at least 2 * slack + 2
 *   slack      0 <= slack <= min(delay_e, delay_i): a block consumes at step s the lists
 *              of step s - slack, so with delayed synapses the NVLink latency is off the
 *              critical path; the last `slack` lists are drained before the launch ends
 *   seq0       exchange sequence number of the launch's first step: the number of steps
 *              exchanged through these inboxes so far.  It only grows (restoring an
 *              earlier simulation step does not rewind it); equal on all ranks
 *   sync       two local int32: [0] status word, zero on entry, BSX_ERR_TIMEOUT after a
 *              wait of more than spin_limit polls (0 = default, about a second) — the
 *              launch then stops at a step boundary and the inboxes must be set up again —
 *              or BSX_ERR_NONFINITE when a neuron's state left the finite range (the
 *              launch stops at the end of that step; the counterpart of the reference's
 *              NaN check, brainstate/transform/_debug.py:282-430, at one compare per neuron);
 *              [1] barrier counter, managed by the call
 * With world = 1 no inbox is read.  All ranks must call with the same steps, step0, seq0.
 */
typedef struct bsx_net_links {
  int32_t world, rank;
  int32_t blocks, words_per_block;
  int64_t words_per_rank;
  int32_t slots, slack;
  int64_t spin_limit;
  int64_t seq0;
  uint64_t* inbox[16];
  int32_t* sync;
  int32_t flags;       /* BSX_LINK_* below; 0 = plainest form (ids pushed after the block's update, header
                          and ids fetched one after the other) */
} bsx_net_links_t;
#define BSX_LINK_EARLY_PUSH 1   /* a warp pushes the ids of its spikes as soon as it has them */
#define BSX_LINK_FETCH_AHEAD 2  /* the receiver fetches a list's header and first 31 ids in one round trip */
#define BSX_LINK_DEFAULT 3
/* Grid every rank must launch for shards of words_per_rank spike words (one block per SM
 * at most, at least one word per warp). */
int bsx_net_shard_geometry(int64_t words_per_rank, int32_t* blocks, int32_t* words_per_block);
size_t bsx_net_inbox_bytes(int32_t world, int32_t blocks, int32_t words_per_block, int32_t slots);
/*
 * Runs steps [step0, step0 + steps) of the shard in ONE cooperative launch: neuron state
 * resident in shared memory (shards of up to about two million neurons; in global memory
 * beyond), one grid-wide barrier per step whatever the delays, the exchange inside the
 * kernel.  Fuses what the reference runs as separate operators per step
 * (examples/400_CUBA_2005_bpu.py:60-66).  raster (may be NULL): (steps, ceil(n_local/32))
 * the RANK's spike words; spike_counts (may be NULL): (steps) spikes of the WHOLE network
 * per step (own count plus the counts of the received lists), overwritten.
 */
int bsx_net_run_sharded(const bsx_net_shard_t* net, const bsx_lif_params_t* params, const bsx_net_links_t* links,
                        int32_t steps, int64_t step0, uint32_t* raster, int32_t* spike_counts,
                        bsx_stream_t stream);
/* Set-up helpers for the buffers above (the only allocating entry points; never on
 * the hot path): allocate zeroed device memory with a 64-byte handle another process
 * on the node can open; open / close a peer's handle; free. */
int bsx_ipc_alloc(size_t bytes, void** ptr, void* handle64);
int bsx_ipc_open(const void* handle64, void** ptr);
int bsx_ipc_close(void* ptr);
int bsx_ipc_free(void* ptr);
/* The hash behind the background drive, on the host (same integer arithmetic). */
uint32_t bsx_drive_hash(uint32_t seed, uint32_t neuron, uint32_t step);

/* ---- small utilities ---------------------------------------------------- */
int bsx_fill_f32(float* dst, int64_t n, float value, bsx_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* BSX_H_ */
