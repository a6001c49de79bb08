// b200mono_moe_ffn_static: the MoE FFN block for callers that cannot allocate.
//
// Some hosts of this library have no way to get device scratch at the moment
// they call it: a serving process that has already handed every free byte of
// HBM to its KV-cache pool (a later cudaMalloc may simply fail), or a thin FFI
// binding that owns plain pointers to inputs and outputs and no allocator at
// all.  For them the block's intermediates live in one fixed array inside the
// library image instead of a caller-provided buffer.  Every GPU that loads the
// library carries those B200MONO_STATIC_SCRATCH_BYTES until the process exits,
// which is why the size is modest and larger problems are refused.
//
// Rules of use
//  * The array's address is looked up once per device (cudaGetSymbolAddress,
//    with that device current) by the first call made on that device.  Make
//    that first call outside any stream capture.
//  * All calls on a device share the array and it keeps whatever the previous
//    call left there.  The words that must start at zero (arrival counter,
//    union count, status) are cleared on the caller's stream before the
//    launches; everything else is written before it is read.
//  * Because the array is shared, two calls whose kernels can overlap on the
//    GPU (different streams, no dependency) race.  Serialise them.
//  * Nothing here calls cudaMalloc, cudaFree or any allocating library routine.
#include <stdio.h>

#include "launch.h"

namespace b200mono {

// Device-resident scratch.  In host code the name `g_static_scratch` is only a handle for the
// runtime's symbol table, not a device address: kernels must be given the pointer that
// cudaGetSymbolAddress returns.
static __device__ __align__(256) unsigned char g_static_scratch[B200MONO_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
static void* g_scratch_ptr[kMaxDevices] = {};

static int static_fail(int code, const char* msg) {
  set_last_error(msg);
  return code;
}

// Address of the array on the current device; resolved on first use per device.
static int scratch_on_current_device(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_fail((int)e, "moe_ffn_static: cudaGetDevice failed");
  if (dev < 0 || dev >= kMaxDevices) return static_fail(B200MONO_E_DEVICE, "moe_ffn_static: device ordinal out of range");
  if (!g_scratch_ptr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || !p) {
      char msg[256];
      snprintf(msg, sizeof(msg), "moe_ffn_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return static_fail(e != cudaSuccess ? (int)e : B200MONO_E_DEVICE, msg);
    }
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return B200MONO_OK;
}

}  // namespace b200mono

using namespace b200mono;

extern "C" int b200mono_moe_ffn_static(const B200MoeFfnArgs* a, void* stream) {
  if (!a) return static_fail(B200MONO_E_ARG, "moe_ffn_static: null args");
  if (a->scratch || a->scratch_bytes)
    return static_fail(B200MONO_E_ARG, "moe_ffn_static: scratch and scratch_bytes must be zero (the library owns the scratch)");
  B200MoeFfnLayout L;
  if (int rc = b200mono_moe_ffn_layout(a->rows, a->hidden, a->inter, a->experts, a->topk, &L)) return rc;
  if (L.total > (int64_t)B200MONO_STATIC_SCRATCH_BYTES) {
    char msg[256];
    snprintf(msg, sizeof(msg),
             "moe_ffn_static: this problem needs %lld bytes of scratch, the built-in array holds %d; "
             "use b200mono_moe_ffn with a caller-provided buffer",
             (long long)L.total, (int)B200MONO_STATIC_SCRATCH_BYTES);
    return static_fail(B200MONO_E_SCRATCH, msg);
  }
  void* scratch = nullptr;
  if (int rc = scratch_on_current_device(&scratch)) return rc;
  // the fixed words at the head of the layout must be zero when the launches start
  const int64_t head = L.res;  // counter, union count and status precede the first data region
  cudaError_t e = cudaMemsetAsync(scratch, 0, (size_t)head, (cudaStream_t)stream);
  if (e != cudaSuccess) {
    char msg[256];
    snprintf(msg, sizeof(msg), "moe_ffn_static: clearing the head words failed: %s", cudaGetErrorString(e));
    return static_fail((int)e, msg);
  }
  B200MoeFfnArgs b = *a;
  b.scratch = scratch;
  b.scratch_bytes = (int64_t)B200MONO_STATIC_SCRATCH_BYTES;
  return b200mono_moe_ffn(&b, stream);
}
