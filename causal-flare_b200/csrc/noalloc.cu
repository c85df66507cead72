// flare_forward_noalloc: the forward entry point for callers that must not allocate device memory.
//
// Who needs it: code that runs where cudaMalloc is off limits - a serving loop that has handed all device
// memory to its own pool, a plugin called from inside another framework's allocator callback or from a
// latency-critical path where an allocation (which may synchronise the device) is unacceptable, or a host
// language binding that has no allocator to offer for the workspace.  flare_forward asks such callers for a
// workspace whenever it splits a long sequence into segments (few (batch, head) lanes); this variant keeps that
// workspace - the per-segment (m, d, u) states of the segment scan - in a fixed array inside the library.
#include <string.h>

#include "flare_common.cuh"

// Capacity of the built-in scratch.  Every GPU that loads the library holds this much memory until exit.
#define FLARE_NOALLOC_SCRATCH_BYTES (8u << 20)

static __device__ __align__(256) unsigned char g_flare_noalloc_scratch[FLARE_NOALLOC_SCRATCH_BYTES];

extern "C" {

size_t flare_noalloc_scratch_capacity(void) { return FLARE_NOALLOC_SCRATCH_BYTES; }

int flare_forward_noalloc(const flare_fwd_args_t* args, flare_stream_t stream) {
  if (args == nullptr) return FLARE_ERR_BAD_POINTER;
  // The array's name is only a host-side handle: the address a kernel can use is asked for here, for the device that
  // is current now, on every call (a lookup in the loaded module, no allocation; nothing is cached, so a context that
  // was torn down and rebuilt, or several host threads, cannot see a stale address).  It is not a stream operation:
  // make the first call on a device before any stream capture.
  void* scratch = nullptr;
  FLARE_CUDA_CHECK(cudaGetSymbolAddress(&scratch, g_flare_noalloc_scratch));
  if (scratch == nullptr) return FLARE_ERR_CUDA;
  flare_fwd_args_t a = *args;
  a.workspace = nullptr;
  a.workspace_bytes = 0;
  size_t need = flare_forward_workspace_bytes(&a);
  if (need > FLARE_NOALLOC_SCRATCH_BYTES && a.dtype == FLARE_F16 && a.path != FLARE_PATH_EXACT) {
    // the tensor-core route of an fp16 call keeps bf16 copies of k and v in the workspace; when those do not fit the
    // built-in scratch the call runs on the exact kernels, which read fp16 directly
    a.path = FLARE_PATH_EXACT;
    need = flare_forward_workspace_bytes(&a);
  }
  if (need > FLARE_NOALLOC_SCRATCH_BYTES) return FLARE_ERR_TOO_LARGE;
  // What must start at zero is cleared by flare_forward itself, on the stream (the gate words of the default path);
  // the segment pass writes every state slot before the scan and the output pass read it.  The rest of the previous
  // call's contents is simply overwritten.
  a.workspace = scratch;
  a.workspace_bytes = FLARE_NOALLOC_SCRATCH_BYTES;
  return flare_forward(&a, stream);
}

}  // extern "C"
