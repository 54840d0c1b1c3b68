// hbsa_forward_static_scratch: the forward for callers that cannot hand us scratch memory.
//
// hbsa_forward needs a small device workspace (block tables, per-row counts, the launch order)
// that the caller normally allocates.  Some hosts have no way to do that at the point of the
// call: a serving process that gave every byte of device memory to its own arena at start-up
// and exposes no allocator to plug-ins, or a plug-in interface whose execute callback receives
// only input and output buffers and forbids cudaMalloc.  For them the same kernels run here on
// a fixed scratch array that lives in the library image, so this entry point calls no
// cudaMalloc, cudaFree or any other allocating routine.
//
// The price: the array is HBSA_STATIC_SCRATCH_BYTES long on every GPU that loads the library,
// for the life of the process; problems whose workspace would not fit are refused; and all
// calls on one GPU share the array, so two calls whose kernels can overlap on the GPU (different
// streams, different threads) race on it - serialise them.
#include <mutex>

#include "hbsa_common.cuh"

namespace {

static __device__ __align__(256) unsigned char g_static_scratch[HBSA_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_mutex;
void* g_scratch_addr[kMaxDevices] = {};   // device address of g_static_scratch, per device ordinal

}  // namespace

extern "C" {

int hbsa_forward_static_scratch(const hbsa_forward_args* args, void* stream) {
  if (!args) {
    hbsa::set_last_error("args is NULL");
    return HBSA_ERR_NULL;
  }
  if (args->struct_bytes != sizeof(hbsa_forward_args)) {
    hbsa::set_last_error("hbsa_forward_args.struct_bytes does not match this library");
    return HBSA_ERR_STRUCT;
  }
  const size_t need = hbsa_workspace_bytes(args->nhead_k, args->num_q_block, args->num_k_block, args->batch);
  if (need == 0) {
    hbsa::set_last_error("nhead_k, num_q_block, num_k_block and batch must be positive");
    return HBSA_ERR_SHAPE;
  }
  if (need > (size_t)HBSA_STATIC_SCRATCH_BYTES) {
    hbsa::set_last_error(
             "this problem needs %zu bytes of scratch but the built-in array holds %zu: "
             "use hbsa_forward with a caller-allocated workspace",
             need, (size_t)HBSA_STATIC_SCRATCH_BYTES);
    return HBSA_ERR_WORKSPACE;
  }

  // Once per device, with that device current: turn the symbol into a device address.  The name
  // g_static_scratch is only a host-side handle here; kernels must be given the looked-up address.
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    hbsa::set_last_error("cudaGetDevice failed or device ordinal out of range: %s",
             cudaGetErrorString(e));
    return e != cudaSuccess ? (int)e : HBSA_ERR_SHAPE;
  }
  void* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (g_scratch_addr[dev] == nullptr) {
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_static_scratch);
      if (e != cudaSuccess || p == nullptr) {
        hbsa::set_last_error("cudaGetSymbolAddress(static scratch) failed: %s", cudaGetErrorString(e));
        return e != cudaSuccess ? (int)e : HBSA_ERR_DRIVER;
      }
      g_scratch_addr[dev] = p;
    }
    scratch = g_scratch_addr[dev];
  }

  // Same kernels as hbsa_forward, on the built-in array.  The schedule kernels clear the status
  // words, the histogram and the bucket cursors at the start of every call, so nothing of the
  // previous call's contents is relied upon.
  hbsa_forward_args local = *args;
  local.workspace = scratch;
  local.workspace_bytes = (size_t)HBSA_STATIC_SCRATCH_BYTES;
  return hbsa_forward(&local, stream);     // its error text is already in hbsa_last_error()
}

}  // extern "C"
