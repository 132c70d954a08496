// Forward attention for callers that are not allowed to allocate device memory.
//
// Some hosts of this library may launch kernels but may not call cudaMalloc (or any
// allocating routine) at the point where attention runs: a plug-in whose execute hook is
// forbidden to allocate, a serving loop that froze its memory budget after warm-up, a
// process that shares the GPU under a fixed reservation.  The regular forward needs an
// operand cache that the caller allocates; here the cache lives in a fixed array that is
// part of the loaded module, so the call needs inputs and outputs only.
//
// Cost and limits: every GPU that loads the library holds the array (FA4B_STATIC_WS_BYTES
// plus alignment slack) until the process exits; shapes whose operand cache is larger are
// rejected; all calls share the one array, so two calls whose kernels overlap on the GPU
// (different streams, or different host threads) race -- serialise them.
#include <mutex>

#include "attn.cuh"

namespace fa4b {

constexpr size_t kStaticWsBytes = FA4B_STATIC_WS_BYTES;
// file-scope scratch; 1 KiB of slack lets the kernels' 1024-byte base alignment be met
static __device__ __align__(256) unsigned char g_static_ws[kStaticWsBytes + 1024];

// Device address of the array for the current device.  In host code `g_static_ws` is only
// a handle for the runtime: the address a kernel may use comes from cudaGetSymbolAddress.
int static_ws_pointer(void** out) {
  static std::mutex mu;
  static void* cached[64] = {};
  int dev = 0;
  FA4B_CUDA(cudaGetDevice(&dev));
  FA4B_REQUIRE(dev >= 0 && dev < 64, FA4B_UNSUPPORTED, "device ordinal %d is beyond the 64 this entry point tracks", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev] == nullptr) {
    void* p = nullptr;
    FA4B_CUDA(cudaGetSymbolAddress(&p, g_static_ws));
    FA4B_REQUIRE(p != nullptr, FA4B_CUDA_ERROR, "cudaGetSymbolAddress returned a NULL address");
    cached[dev] = reinterpret_cast<void*>((reinterpret_cast<uintptr_t>(p) + 1023) & ~uintptr_t(1023));
  }
  *out = cached[dev];
  return FA4B_OK;
}

}  // namespace fa4b

using namespace fa4b;

extern "C" int fa4b_attn_fwd_static(const fa4b_attn_fwd_args* a, void* stream) {
  FA4B_REQUIRE(a != nullptr, FA4B_BAD_ARG, "args is NULL");
  if (int s = check_dims(a->dims)) return s;
  // the forward touches the saved section of the layout only (operands, amax and status words)
  const size_t need = make_ws_layout(a->dims).saved_total;
  FA4B_REQUIRE(need <= kStaticWsBytes, FA4B_BAD_SHAPE,
               "this shape needs an operand cache of %zu bytes; the built-in scratch holds %zu (FA4B_STATIC_WS_BYTES): "
               "use fa4b_attn_fwd with a caller-allocated workspace",
               need, kStaticWsBytes);
  void* ws = nullptr;
  if (int s = static_ws_pointer(&ws)) return s;
  fa4b_attn_fwd_args call = *a;
  call.ws = ws;
  // the array still holds the previous call's operands: always publish again; the publication
  // step clears the amax words and the status words it depends on
  call.prepared = 0;
  return launch_attn_fwd(call, static_cast<cudaStream_t>(stream));
}
