// extern "C" entry points of libhbsattn_b200 (declared in include/hbsattn_b200.h).
#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include "hbsa_common.cuh"

namespace {

thread_local char g_err[512] = "";

int fail(int code, const char* msg) {
  snprintf(g_err, sizeof(g_err), "%s", msg);
  return code;
}

int fail_cuda(cudaError_t e, const char* where) {
  snprintf(g_err, sizeof(g_err), "%s: %s", where, cudaGetErrorString(e));
  return (int)e;
}

// Validates everything that does not need the device and fills the kernel-side description.
int make_problem(const hbsa_forward_args* a, bool need_tensors, hbsa::Problem* p) {
  if (!a) return fail(HBSA_ERR_NULL, "args is NULL");
  if (a->struct_bytes != sizeof(hbsa_forward_args)) return fail(HBSA_ERR_STRUCT, "hbsa_forward_args.struct_bytes does not match this library");
  if (!a->cu_q_seqlens || !a->cu_k_seqlens || !a->workspace)
    return fail(HBSA_ERR_NULL, "cu_q_seqlens, cu_k_seqlens and workspace must not be NULL");
  if ((a->csr_row_ptr == nullptr) != (a->csr_col_idx == nullptr))
    return fail(HBSA_ERR_NULL, "csr_row_ptr and csr_col_idx must be given together");
  if (!a->block_mask && !a->csr_row_ptr) return fail(HBSA_ERR_NULL, "either block_mask or the CSR block mask must be given");
  if (need_tensors && (!a->q || !a->k || !a->v || !a->o)) return fail(HBSA_ERR_NULL, "q, k, v and o must not be NULL");
  if (a->batch <= 0 || a->nhead_q <= 0 || a->nhead_k <= 0 || a->headdim <= 0 || a->num_q_block <= 0 ||
      a->num_k_block <= 0 || a->total_q < 0 || a->total_k < 0)
    return fail(HBSA_ERR_SHAPE, "batch, head counts, headdim and block counts must be positive");
  if (a->nhead_q % a->nhead_k != 0) return fail(HBSA_ERR_SHAPE, "nhead_q must be divisible by nhead_k (for GQA)");
  if (a->headdim > 256) return fail(HBSA_ERR_SHAPE, "headdim above 256 is not supported");
  if (a->q_block_size <= 0 || a->k_block_size <= 0 || a->q_block_size % 16 != 0 || a->k_block_size % 16 != 0)
    return fail(HBSA_ERR_BLOCK_SIZE, "q_block_size and k_block_size must be integer multiples of 16.");
  if (a->dtype != HBSA_DTYPE_BF16 && a->dtype != HBSA_DTYPE_F16 && a->dtype != HBSA_DTYPE_F32)
    return fail(HBSA_ERR_DTYPE, "unknown dtype");
  if (a->impl != HBSA_IMPL_AUTO && a->impl != HBSA_IMPL_GENERIC && a->impl != HBSA_IMPL_SM100)
    return fail(HBSA_ERR_DTYPE, "unknown impl");
  if (a->workspace_bytes < hbsa::workspace_bytes(a->nhead_k, a->num_q_block, a->num_k_block, a->batch))
    return fail(HBSA_ERR_WORKSPACE, "workspace is smaller than hbsa_workspace_bytes()");
  if (((uintptr_t)a->workspace) % 256 != 0) return fail(HBSA_ERR_WORKSPACE, "workspace must be 256-byte aligned");
  p->cu_q = a->cu_q_seqlens;
  p->cu_k = a->cu_k_seqlens;
  p->mask = a->csr_row_ptr ? nullptr : a->block_mask;       // a CSR mask takes precedence
  p->csr_ptr = a->csr_row_ptr;
  p->csr_idx = a->csr_col_idx;
  p->mask_s0 = a->mask_stride[0];
  p->mask_s1 = a->mask_stride[1];
  p->mask_s2 = a->mask_stride[2];
  p->batch = a->batch;
  p->nhead_q = a->nhead_q;
  p->nhead_k = a->nhead_k;
  p->group = a->nhead_q / a->nhead_k;
  p->headdim = a->headdim;
  p->num_q_block = a->num_q_block;
  p->num_k_block = a->num_k_block;
  p->qbs = a->q_block_size;
  p->kbs = a->k_block_size;
  p->causal = a->causal ? 1 : 0;
  p->scale = a->use_default_scale ? 1.0f / sqrtf((float)a->headdim) : a->softmax_scale;
  p->kv_tile = hbsa::sm100_kv_tile_rows(a->k_block_size);
  return 0;
}

int select_impl(const hbsa_forward_args* a, const hbsa::Problem& p) {
  const char* why = hbsa::sm100_ineligible_reason(*a, p.scale);
  if (a->impl == HBSA_IMPL_GENERIC) return HBSA_IMPL_GENERIC;
  if (a->impl == HBSA_IMPL_SM100) {
    if (why) {
      snprintf(g_err, sizeof(g_err), "the tcgen05 kernel cannot run this problem: %s", why);
      return HBSA_ERR_UNSUPPORTED;
    }
    return HBSA_IMPL_SM100;
  }
  return why ? HBSA_IMPL_GENERIC : HBSA_IMPL_SM100;
}

}  // namespace

namespace hbsa {
void set_last_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}
}  // namespace hbsa

extern "C" {

int hbsa_version(void) { return HBSA_ABI_VERSION; }

const char* hbsa_last_error(void) { return g_err; }

int hbsa_calculate_blocks(const int32_t* cu_seqlen, int batch, int block_size, int capacity, int32_t* cu_block,
                          int32_t* block_to_batch, int32_t* cu_num_block, void* stream) {
  if (!cu_seqlen || !cu_num_block) return fail(HBSA_ERR_NULL, "cu_seqlen and cu_num_block must not be NULL");
  if (batch <= 0 || capacity < 0) return fail(HBSA_ERR_SHAPE, "batch must be positive and capacity non-negative");
  if (block_size <= 0) return fail(HBSA_ERR_BLOCK_SIZE, "block_size must be positive");
  cudaError_t e = hbsa::launch_calculate_blocks(cu_seqlen, batch, block_size, capacity, capacity > 0 ? cu_block : nullptr,
                                                capacity > 0 ? block_to_batch : nullptr, cu_num_block,
                                                static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? 0 : fail_cuda(e, "hbsa_calculate_blocks");
}

size_t hbsa_workspace_bytes(int nhead_k, int num_q_block, int num_k_block, int batch) {
  if (nhead_k <= 0 || num_q_block <= 0 || num_k_block <= 0 || batch <= 0) return 0;
  return hbsa::workspace_bytes(nhead_k, num_q_block, num_k_block, batch);
}

int hbsa_select_impl(const hbsa_forward_args* args) {
  hbsa::Problem p;
  int rc = make_problem(args, true, &p);
  if (rc != 0) return rc;
  return select_impl(args, p);
}

int hbsa_build_schedule(const hbsa_forward_args* args, void* stream_) {
  hbsa::Problem p;
  int rc = make_problem(args, false, &p);
  if (rc != 0) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  hbsa::Workspace ws = hbsa::make_workspace(args->workspace, p.nhead_k, p.num_q_block, p.num_k_block, p.batch);
  cudaError_t e = hbsa::launch_schedule(p, ws, nullptr, stream);
  return e == cudaSuccess ? 0 : fail_cuda(e, "hbsa_build_schedule");
}

int hbsa_attention(const hbsa_forward_args* args, void* stream_) {
  hbsa::Problem p;
  int rc = make_problem(args, true, &p);
  if (rc != 0) return rc;
  const int impl = select_impl(args, p);
  if (impl < 0) return impl;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  hbsa::Workspace ws = hbsa::make_workspace(args->workspace, p.nhead_k, p.num_q_block, p.num_k_block, p.batch);
  if (impl == HBSA_IMPL_SM100) {
    const char* text = "";
    rc = hbsa::launch_forward_sm100(p, ws, *args, stream, &text);
    return rc != 0 ? fail(rc, text) : 0;
  }
  cudaError_t e = hbsa::launch_forward_generic(p, ws, *args, stream);
  return e == cudaSuccess ? 0 : fail_cuda(e, "hbsa_attention (generic kernel)");
}

int hbsa_forward(const hbsa_forward_args* args, void* stream) {
  hbsa::Problem p;
  int rc = make_problem(args, true, &p);          // reject everything before the first launch
  if (rc != 0) return rc;
  rc = select_impl(args, p);
  if (rc < 0) return rc;
  rc = hbsa_build_schedule(args, stream);
  if (rc != 0) return rc;
  return hbsa_attention(args, stream);
}

int hbsa_block_decisions(const hbsa_forward_args* args, uint8_t* decisions, int32_t* counts, void* stream_) {
  hbsa::Problem p;
  int rc = make_problem(args, false, &p);
  if (rc != 0) return rc;
  if (!decisions && !counts) return fail(HBSA_ERR_NULL, "decisions and counts must not both be NULL");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  hbsa::Workspace ws = hbsa::make_workspace(args->workspace, p.nhead_k, p.num_q_block, p.num_k_block, p.batch);
  cudaError_t e = cudaSuccess;
  if (decisions) e = cudaMemsetAsync(decisions, 0, (size_t)p.nhead_k * p.num_q_block * p.num_k_block, stream);
  if (e != cudaSuccess) return fail_cuda(e, "hbsa_block_decisions (memset)");
  e = hbsa::launch_schedule(p, ws, decisions, stream);
  if (e != cudaSuccess) return fail_cuda(e, "hbsa_block_decisions");
  if (counts) {
    e = cudaMemcpyAsync(counts, ws.counts, (size_t)p.nhead_k * p.num_q_block * sizeof(int32_t), cudaMemcpyDeviceToDevice, stream);
    if (e != cudaSuccess) return fail_cuda(e, "hbsa_block_decisions (counts)");
  }
  return 0;
}

size_t hbsa_backward_workspace_bytes(int64_t total_q, int64_t total_k, int nhead_q, int nhead_k, int headdim) {
  if (total_q < 0 || total_k < 0 || nhead_q <= 0 || nhead_k <= 0 || headdim <= 0) return 0;
  return hbsa::backward_workspace_bytes(total_q, total_k, nhead_q, nhead_k, headdim);
}

int hbsa_backward(const hbsa_backward_args* b, void* stream_) {
  if (!b) return fail(HBSA_ERR_NULL, "args is NULL");
  if (b->struct_bytes != sizeof(hbsa_backward_args)) return fail(HBSA_ERR_STRUCT, "hbsa_backward_args.struct_bytes does not match this library");
  hbsa::Problem p;
  int rc = make_problem(&b->fwd, true, &p);
  if (rc != 0) return rc;
  if (!b->d_o || !b->dq || !b->dk || !b->dv || !b->grad_workspace) return fail(HBSA_ERR_NULL, "d_o, dq, dk, dv and grad_workspace must not be NULL");
  if (!b->fwd.lse) return fail(HBSA_ERR_NULL, "the backward needs the lse of the forward (hbsa_forward_args.lse)");
  if (b->grad_workspace_bytes < hbsa::backward_workspace_bytes(b->fwd.total_q, b->fwd.total_k, b->fwd.nhead_q, b->fwd.nhead_k, b->fwd.headdim))
    return fail(HBSA_ERR_WORKSPACE, "grad_workspace is smaller than hbsa_backward_workspace_bytes()");
  if (((uintptr_t)b->grad_workspace) % 256 != 0) return fail(HBSA_ERR_WORKSPACE, "grad_workspace must be 256-byte aligned");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  hbsa::Workspace ws = hbsa::make_workspace(b->fwd.workspace, p.nhead_k, p.num_q_block, p.num_k_block, p.batch);
  cudaError_t e = hbsa::launch_schedule(p, ws, nullptr, stream);
  if (e != cudaSuccess) return fail_cuda(e, "hbsa_backward (schedule)");
  e = hbsa::launch_backward_generic(p, ws, *b, stream);
  return e == cudaSuccess ? 0 : fail_cuda(e, "hbsa_backward");
}

size_t hbsa_debug_trace_bytes(void) { return hbsa::sm100_trace_bytes(); }

void hbsa_debug_set_trace(void* device_buffer) { hbsa::sm100_set_trace(static_cast<long long*>(device_buffer)); }

void hbsa_debug_set_wait_budget(long long clocks, int stall_producer) { hbsa::sm100_set_wait_budget(clocks, stall_producer); }

int hbsa_read_status(const void* workspace, int32_t* status_out, void* stream_) {
  if (!workspace || !status_out) return fail(HBSA_ERR_NULL, "workspace and status_out must not be NULL");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  cudaError_t e = cudaMemcpyAsync(status_out, workspace, hbsa::kStatusWords * sizeof(int32_t), cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  return e == cudaSuccess ? 0 : fail_cuda(e, "hbsa_read_status");
}

}  // extern "C"
