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
//
// The very first call on a device is special: it asks the CUDA runtime for the device address of
// the array, and with lazy module loading that is the moment the driver loads this library's device
// code and places the array in device memory.  Do it once at start-up, outside any stream capture;
// every later call on that device touches no allocator at all.
#include <mutex>

#include "hbsa_common.cuh"

namespace {

static __device__ __align__(256) unsigned char g_static_scratch[HBSA_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_mutex;
void* g_scratch_addr[kMaxDevices] = {};   // device address of g_static_scratch, per device ordinal

}  // namespace

// Device address of the built-in array on the current device (looked up once per device), or NULL with the
// error text set.  `rc` receives the code to return on failure.
static void* static_scratch_address(int* rc) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    hbsa::set_last_error("cudaGetDevice failed or device ordinal out of range: %s", cudaGetErrorString(e));
    *rc = e != cudaSuccess ? (int)e : HBSA_ERR_SHAPE;
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_scratch_addr[dev] == nullptr) {
    // The name g_static_scratch is only a host-side handle here; kernels must be given the looked-up address.
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || p == nullptr) {
      hbsa::set_last_error("cudaGetSymbolAddress(static scratch) failed: %s", cudaGetErrorString(e));
      *rc = e != cudaSuccess ? (int)e : HBSA_ERR_DRIVER;
      return nullptr;
    }
    g_scratch_addr[dev] = p;
  }
  return g_scratch_addr[dev];
}

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

  // Once per device, with that device current: turn the symbol into a device address.
  int rc = 0;
  void* scratch = static_scratch_address(&rc);
  if (scratch == nullptr) return rc;

  // Same kernels as hbsa_forward, on the built-in array.  The first schedule kernel of every call
  // clears the status words and the work-cursor block (next item, count of CTAs that have left) and
  // every table the attention kernel reads is rewritten for this call's sizes, so nothing of the
  // previous call's contents is relied upon - whether that call was larger or smaller.
  hbsa_forward_args local = *args;
  local.workspace = scratch;
  local.workspace_bytes = (size_t)HBSA_STATIC_SCRATCH_BYTES;
  return hbsa_forward(&local, stream);     // its error text is already in hbsa_last_error()
}

int hbsa_static_scratch_status(int32_t* status_out, void* stream_) {
  if (!status_out) {
    hbsa::set_last_error("status_out must not be NULL");
    return HBSA_ERR_NULL;
  }
  int rc = 0;
  void* scratch = static_scratch_address(&rc);
  if (scratch == nullptr) return rc;
  // The status words are the first words of the array, exactly as in a caller-owned workspace.
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  cudaError_t e = cudaMemcpyAsync(status_out, scratch, hbsa::kStatusWords * sizeof(int32_t), cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) {
    hbsa::set_last_error("hbsa_static_scratch_status: %s", cudaGetErrorString(e));
    return (int)e;
  }
  return 0;
}

}  // extern "C"
