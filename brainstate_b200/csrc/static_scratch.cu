// Event vecmat for callers that cannot hand over a workspace.
//
// bsx_event_vecmat needs a queue of active rows in global memory and asks the
// caller for it.  Some callers have no way to get device memory at the moment
// they call: a custom-call handler running inside a framework that has already
// claimed the GPU's memory for its own pool (a cudaMalloc there can fail, or
// stall the whole device while it runs), and code on a latency-critical path
// that must not hit the implicit device-wide synchronisation of an allocation.
// For them the queue lives in a fixed array that is part of this library's
// image: every GPU that loads the library carries these 4 MiB until the process
// exits, whether or not the entry point is ever called.
#include <atomic>

#include "common.cuh"
#include "internal.cuh"

namespace bsx {

// Queue header + one 32-bit entry per (batch row, presynaptic neuron).
constexpr size_t kStaticQueueBytes = size_t(4) << 20;
static __device__ __align__(256) unsigned char g_static_queue[kStaticQueueBytes];

// In host code `g_static_queue` is only a handle for the runtime, not an address
// a kernel may dereference; the device address is looked up once per device and
// kept here.
constexpr int kMaxDevices = 64;
static std::atomic<void*> g_static_queue_addr[kMaxDevices];

static int static_queue_address(void** out) {
  int dev = 0;
  BSX_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(BSX_ERR_UNSUPPORTED, "device ordinal %d above %d", dev, kMaxDevices - 1);
  void* p = g_static_queue_addr[dev].load(std::memory_order_acquire);
  if (!p) {
    // First use on this device (it is the current one): resolve the symbol.
    BSX_CUDA(cudaGetSymbolAddress(&p, g_static_queue));
    if (!p) return fail(BSX_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
    g_static_queue_addr[dev].store(p, std::memory_order_release);
  }
  *out = p;
  return BSX_OK;
}

}  // namespace bsx

using namespace bsx;

extern "C" int bsx_event_vecmat_static(const bsx_conn_t* conn, const void* spikes, int spike_format,
                                       int64_t batch, float* out, int accumulate, bsx_stream_t stream) {
  BSX_TRACE("bsx_event_vecmat_static");
  if (spike_format < BSX_SPK_BOOL8 || spike_format > BSX_SPK_LIST)
    return fail(BSX_ERR_INVALID_ARG, "unknown spike format %d", spike_format);
  if (!conn) return fail(BSX_ERR_INVALID_ARG, "conn is NULL");
  if (batch < 0 || conn->n_pre < 0) return fail(BSX_ERR_INVALID_ARG, "negative size");
  const size_t need = bsx_event_vecmat_workspace_bytes(batch, conn->n_pre);
  if (spike_format != BSX_SPK_LIST &&
      ((double)batch * (double)conn->n_pre > (double)BSX_STATIC_QUEUE_MAX_SPIKES || need > kStaticQueueBytes))
    return fail(BSX_ERR_WORKSPACE,
                "bsx_event_vecmat_static: batch * n_pre = %.0f exceeds the built-in queue of %d entries; "
                "use bsx_event_vecmat with a caller-provided workspace",
                (double)batch * (double)conn->n_pre, BSX_STATIC_QUEUE_MAX_SPIKES);
  void* queue = nullptr;
  int rc = static_queue_address(&queue);
  if (rc) return rc;
  // The queue keeps whatever the previous call left in it.  The only word that must
  // start at zero is the entry counter in its header, which the compaction step
  // clears on the stream before it counts; entries beyond the counter are never read.
  return vecmat_common(conn, spikes, spike_format, nullptr, batch, out, accumulate, queue, kStaticQueueBytes, 0, 0,
                       as_stream(stream));
}
