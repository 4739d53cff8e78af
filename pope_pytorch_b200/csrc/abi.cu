// extern "C" boundary of libpope_b200.so: argument validation and dispatch.
// Declarations and the contract of each entry point live in include/pope_b200.h.
#include <cstdlib>

#include "kernels.h"

namespace {

thread_local const char* g_last_path = "none";

int check_device() {
  // one lookup per host thread and device: the kernels are sm_100a only
  static thread_local int cached_dev = -1, cached_ok = 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return POPE_ERR_CUDA;
  if (dev != cached_dev) {
    int major = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return POPE_ERR_CUDA;
    cached_dev = dev, cached_ok = (major == 10);
  }
  return cached_ok ? POPE_OK : POPE_ERR_ARCH;
}

int check_shape(const PopeShape& s) {
  if (s.B <= 0 || s.H <= 0 || s.Hk <= 0 || s.Nq <= 0 || s.Nk <= 0 || s.d <= 0 || s.r < 0) return POPE_ERR_BAD_ARG;
  if (s.H % s.Hk != 0 || s.Nq > s.Nk || s.r > s.d) return POPE_ERR_BAD_ARG;
  if (s.dtype != POPE_F32 && s.dtype != POPE_BF16 && s.dtype != POPE_F16) return POPE_ERR_BAD_ARG;
  if ((int64_t)s.B * s.H > 65535) return POPE_ERR_UNSUPPORTED;
  return POPE_OK;
}

// POPE_B200_FORCE_SIMT=1 routes every call to the exact-arithmetic family (for A/B comparisons)
bool force_simt() {
  const char* e = std::getenv("POPE_B200_FORCE_SIMT");
  return e && e[0] == '1';
}

int check_embed(const PopeShape& s, const PopeEmbed& e) {
  if (s.r > 0 && (!e.freqs || !e.bias)) return POPE_ERR_BAD_ARG;
  return POPE_OK;
}

}  // namespace

namespace pope {
void note_last_path(const char* family) { g_last_path = family; }
}  // namespace pope

extern "C" {

int pope_b200_abi_version(void) { return POPE_B200_ABI_VERSION; }

const char* pope_b200_status_str(int status) {
  switch (status) {
    case POPE_OK: return "ok";
    case POPE_ERR_BAD_ARG: return "bad argument (null pointer, size, Nq > Nk, r > d, H % Hk != 0, struct size)";
    case POPE_ERR_UNSUPPORTED: return "unsupported shape or dtype";
    case POPE_ERR_MISALIGNED: return "misaligned pointer or stride";
    case POPE_ERR_WORKSPACE: return "workspace missing or too small";
    case POPE_ERR_CUDA: return "CUDA runtime error";
    case POPE_ERR_ARCH: return "device is not compute capability 10.x (B200)";
    case POPE_ERR_TOO_LARGE: return "problem exceeds the library's fixed built-in scratch capacity";
    default: return "unknown status";
  }
}

const char* pope_b200_last_path(void) { return g_last_path; }

int pope_b200_device_status(void) { return static_cast<int>(pope::tc_read_status()); }

int pope_b200_clear_device_status(void) { return pope::tc_clear_status() == cudaSuccess ? POPE_OK : POPE_ERR_CUDA; }

int pope_b200_selftest_bounded_wait(void* stream) {
  int rc = check_device();
  if (rc != POPE_OK) return rc;
  return pope::tc_selftest_bounded_wait(static_cast<cudaStream_t>(stream)) == cudaSuccess ? POPE_OK : POPE_ERR_CUDA;
}

size_t pope_b200_workspace_bytes(int op, const void* args) {
  if (!args) return 0;
  switch (op) {
    case POPE_OP_SIM_FWD: {
      const PopeSimArgs& a = *static_cast<const PopeSimArgs*>(args);
      if (a.struct_bytes != sizeof(PopeSimArgs) || check_shape(a.shape) != POPE_OK) return 0;
      return (!force_simt() && pope::sim_fwd_tc_supported(a)) ? pope::sim_fwd_tc_workspace(a) : 0;
    }
    case POPE_OP_SIM_BWD: {
      const PopeSimBwdArgs& a = *static_cast<const PopeSimBwdArgs*>(args);
      if (a.struct_bytes != sizeof(PopeSimBwdArgs) || check_shape(a.shape) != POPE_OK) return 0;
      return (!force_simt() && pope::sim_bwd_tc_supported(a)) ? pope::sim_bwd_tc_workspace(a) : 0;
    }
    case POPE_OP_ATTN_FWD: {
      const PopeAttnArgs& a = *static_cast<const PopeAttnArgs*>(args);
      if (a.struct_bytes != sizeof(PopeAttnArgs) || check_shape(a.shape) != POPE_OK) return 0;
      if (!force_simt() && pope::attn_fwd_tc_supported(a)) return pope::attn_fwd_tc_workspace(a);
      if (!force_simt() && pope::decode_stream_supported(a)) return pope::decode_stream_workspace(a);
      return pope::attn_fwd_simt_workspace(a);
    }
    case POPE_OP_ATTN_BWD: {
      const PopeAttnBwdArgs& a = *static_cast<const PopeAttnBwdArgs*>(args);
      if (a.struct_bytes != sizeof(PopeAttnBwdArgs) || check_shape(a.shape) != POPE_OK) return 0;
      if (!force_simt() && pope::attn_bwd_tc_supported(a)) return pope::attn_bwd_tc_workspace(a);
      return pope::attn_bwd_simt_workspace(a);
    }
    case POPE_OP_DECODE_PAGED: {
      const PopePagedDecodeArgs& a = *static_cast<const PopePagedDecodeArgs*>(args);
      if (a.struct_bytes != sizeof(PopePagedDecodeArgs) || check_shape(a.shape) != POPE_OK) return 0;
      return pope::decode_paged_supported(a) ? pope::decode_paged_workspace(a) : 0;
    }
    default: return 0;
  }
}

int pope_b200_sim_fwd(const PopeSimArgs* a, void* stream) {
  if (!a || a->struct_bytes != sizeof(PopeSimArgs)) return POPE_ERR_BAD_ARG;
  int rc = check_shape(a->shape);
  if (rc == POPE_OK) rc = check_embed(a->shape, a->embed);
  if (rc != POPE_OK) return rc;
  if (!a->q || !a->k || !a->sim) return POPE_ERR_BAD_ARG;
  // the tensor-core kernel needs its phase tables; a caller that passes no workspace gets the exact family
  const bool tc = !force_simt() && pope::sim_fwd_tc_supported(*a) && a->workspace &&
                  a->workspace_bytes >= pope::sim_fwd_tc_workspace(*a) &&
                  (reinterpret_cast<uintptr_t>(a->workspace) & 15) == 0;
  if ((rc = check_device()) != POPE_OK) return rc;
  const cudaStream_t st = static_cast<cudaStream_t>(stream);
  if ((tc ? pope::sim_fwd_tc(*a, st) : pope::sim_fwd_simt(*a, st)) != cudaSuccess) return POPE_ERR_CUDA;
  g_last_path = tc ? "tcgen05" : "simt";
  return POPE_OK;
}

int pope_b200_sim_bwd(const PopeSimBwdArgs* a, void* stream) {
  if (!a || a->struct_bytes != sizeof(PopeSimBwdArgs)) return POPE_ERR_BAD_ARG;
  int rc = check_shape(a->shape);
  if (rc == POPE_OK) rc = check_embed(a->shape, a->embed);
  if (rc != POPE_OK) return rc;
  if (!a->q || !a->k || !a->dsim || !a->dq || !a->dk) return POPE_ERR_BAD_ARG;
  // the tensor-core kernels need the operand images; a caller that passes no workspace gets the exact family
  const bool tc = !force_simt() && pope::sim_bwd_tc_supported(*a) && a->workspace &&
                  a->workspace_bytes >= pope::sim_bwd_tc_workspace(*a) && (reinterpret_cast<uintptr_t>(a->workspace) & 15) == 0;
  if ((rc = check_device()) != POPE_OK) return rc;
  const cudaStream_t st = static_cast<cudaStream_t>(stream);
  if ((tc ? pope::sim_bwd_tc(*a, st) : pope::sim_bwd_simt(*a, st)) != cudaSuccess) return POPE_ERR_CUDA;
  g_last_path = tc ? "tcgen05" : "simt";
  return POPE_OK;
}

int pope_b200_attn_fwd(const PopeAttnArgs* a, void* stream) {
  if (!a || a->struct_bytes != sizeof(PopeAttnArgs)) return POPE_ERR_BAD_ARG;
  int rc = check_shape(a->shape);
  if (rc == POPE_OK) rc = check_embed(a->shape, a->embed);
  if (rc != POPE_OK) return rc;
  if (!a->q || !a->k || !a->v || !a->out || !a->lse) return POPE_ERR_BAD_ARG;
  if (a->shape.d > 256) return POPE_ERR_UNSUPPORTED;
  const bool tc = !force_simt() && pope::attn_fwd_tc_supported(*a);
  const bool dec = !tc && !force_simt() && pope::decode_stream_supported(*a);
  const size_t need = tc ? pope::attn_fwd_tc_workspace(*a) : dec ? pope::decode_stream_workspace(*a) : pope::attn_fwd_simt_workspace(*a);
  if (need > 0 && (!a->workspace || a->workspace_bytes < need)) return POPE_ERR_WORKSPACE;
  if (need > 0 && (reinterpret_cast<uintptr_t>(a->workspace) & 15) != 0) return POPE_ERR_MISALIGNED;
  if ((rc = check_device()) != POPE_OK) return rc;
  const cudaStream_t st = static_cast<cudaStream_t>(stream);
  const cudaError_t e = tc ? pope::attn_fwd_tc(*a, st) : dec ? pope::decode_stream(*a, st) : pope::attn_fwd_simt(*a, st);
  if (e != cudaSuccess) return POPE_ERR_CUDA;
  g_last_path = tc ? "tcgen05" : dec ? "decode_stream" : "simt";
  return POPE_OK;
}

int pope_b200_attn_bwd(const PopeAttnBwdArgs* a, void* stream) {
  if (!a || a->struct_bytes != sizeof(PopeAttnBwdArgs)) return POPE_ERR_BAD_ARG;
  int rc = check_shape(a->shape);
  if (rc == POPE_OK) rc = check_embed(a->shape, a->embed);
  if (rc != POPE_OK) return rc;
  if (!a->q || !a->k || !a->v || !a->out || !a->dout || !a->lse || !a->dq || !a->dk || !a->dv) return POPE_ERR_BAD_ARG;
  if (a->shape.d > 256) return POPE_ERR_UNSUPPORTED;
  const bool tc = !force_simt() && pope::attn_bwd_tc_supported(*a);
  const size_t need = tc ? pope::attn_bwd_tc_workspace(*a) : pope::attn_bwd_simt_workspace(*a);
  if (!a->workspace || a->workspace_bytes < need) return POPE_ERR_WORKSPACE;
  if ((reinterpret_cast<uintptr_t>(a->workspace) & 15) != 0) return POPE_ERR_MISALIGNED;
  if ((rc = check_device()) != POPE_OK) return rc;
  const cudaStream_t st = static_cast<cudaStream_t>(stream);
  if ((tc ? pope::attn_bwd_tc(*a, st) : pope::attn_bwd_simt(*a, st)) != cudaSuccess) return POPE_ERR_CUDA;
  g_last_path = tc ? "tcgen05" : "simt";
  return POPE_OK;
}

static bool rows_on_8_bytes(const float* ptr, const PopeStride3& st) {
  return (reinterpret_cast<uintptr_t>(ptr) & 7) == 0 && st.b % 2 == 0 && st.h % 2 == 0 && st.n % 2 == 0;
}

int pope_b200_apply_qk_fwd(const PopeApplyArgs* a, void* stream) {
  if (!a || a->struct_bytes != sizeof(PopeApplyArgs)) return POPE_ERR_BAD_ARG;
  int rc = check_shape(a->shape);
  if (rc == POPE_OK) rc = check_embed(a->shape, a->embed);
  if (rc != POPE_OK) return rc;
  if (!a->q || !a->k || !a->q_out || !a->k_out) return POPE_ERR_BAD_ARG;
  if (a->shape.d > 256) return POPE_ERR_UNSUPPORTED;
  if (!rows_on_8_bytes(a->q_out, a->sqo) || !rows_on_8_bytes(a->k_out, a->sko)) return POPE_ERR_MISALIGNED;
  if ((rc = check_device()) != POPE_OK) return rc;
  if (pope::apply_qk_fwd(*a, static_cast<cudaStream_t>(stream)) != cudaSuccess) return POPE_ERR_CUDA;
  g_last_path = "simt";
  return POPE_OK;
}

int pope_b200_apply_qk_bwd(const PopeApplyBwdArgs* a, void* stream) {
  if (!a || a->struct_bytes != sizeof(PopeApplyBwdArgs)) return POPE_ERR_BAD_ARG;
  int rc = check_shape(a->shape);
  if (rc == POPE_OK) rc = check_embed(a->shape, a->embed);
  if (rc != POPE_OK) return rc;
  if (!a->q || !a->k || !a->dq_out || !a->dk_out || !a->dq || !a->dk) return POPE_ERR_BAD_ARG;
  if (a->shape.d > 256) return POPE_ERR_UNSUPPORTED;
  if (!rows_on_8_bytes(a->dq_out, a->sdqo) || !rows_on_8_bytes(a->dk_out, a->sdko)) return POPE_ERR_MISALIGNED;
  if ((rc = check_device()) != POPE_OK) return rc;
  if (pope::apply_qk_bwd(*a, static_cast<cudaStream_t>(stream)) != cudaSuccess) return POPE_ERR_CUDA;
  g_last_path = "simt";
  return POPE_OK;
}

static int check_paged(const PopePagedKV& kv, int B) {
  if (!kv.k_pages || !kv.v_pages || !kv.page_table || !kv.seq_lens) return POPE_ERR_BAD_ARG;
  if (kv.num_pages <= 0 || kv.page_size <= 0 || kv.max_pages_per_seq <= 0 || B <= 0) return POPE_ERR_BAD_ARG;
  if (kv.page_size % 64 != 0) return POPE_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(kv.k_pages) & 15) != 0 || (reinterpret_cast<uintptr_t>(kv.v_pages) & 15) != 0) return POPE_ERR_MISALIGNED;
  return POPE_OK;
}

int pope_b200_kv_append(const PopeKvAppendArgs* a, void* stream) {
  if (!a || a->struct_bytes != sizeof(PopeKvAppendArgs)) return POPE_ERR_BAD_ARG;
  if (a->B <= 0 || a->Hk <= 0 || a->d <= 0 || a->n_new < 0 || !a->k || !a->v) return POPE_ERR_BAD_ARG;
  if (a->dtype != POPE_BF16 && a->dtype != POPE_F16) return POPE_ERR_UNSUPPORTED;
  if (a->d % 8 != 0 || a->Hk > 65535 || a->B > 65535) return POPE_ERR_UNSUPPORTED;
  int rc = check_paged(a->kv, a->B);
  if (rc != POPE_OK) return rc;
  auto rows16 = [](const void* ptr, const PopeStride3& st) {
    return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0 && st.b % 8 == 0 && st.h % 8 == 0 && st.n % 8 == 0;
  };
  if (!rows16(a->k, a->sk) || !rows16(a->v, a->sv)) return POPE_ERR_MISALIGNED;
  if (a->n_new == 0) return POPE_OK;
  if ((rc = check_device()) != POPE_OK) return rc;
  if (pope::kv_append(*a, static_cast<cudaStream_t>(stream)) != cudaSuccess) return POPE_ERR_CUDA;
  g_last_path = "kv_append";
  return POPE_OK;
}

int pope_b200_attn_decode_paged(const PopePagedDecodeArgs* a, void* stream) {
  if (!a || a->struct_bytes != sizeof(PopePagedDecodeArgs)) return POPE_ERR_BAD_ARG;
  int rc = check_shape(a->shape);
  if (rc == POPE_OK) rc = check_embed(a->shape, a->embed);
  if (rc == POPE_OK) rc = check_paged(a->kv, a->shape.B);
  if (rc != POPE_OK) return rc;
  if (!a->q || !a->out) return POPE_ERR_BAD_ARG;
  if (!pope::decode_paged_supported(*a)) return POPE_ERR_UNSUPPORTED;
  const size_t need = pope::decode_paged_workspace(*a);
  if (!a->workspace || a->workspace_bytes < need) return POPE_ERR_WORKSPACE;
  if ((reinterpret_cast<uintptr_t>(a->workspace) & 15) != 0) return POPE_ERR_MISALIGNED;
  if ((rc = check_device()) != POPE_OK) return rc;
  if (pope::decode_paged(*a, static_cast<cudaStream_t>(stream)) != cudaSuccess) return POPE_ERR_CUDA;
  g_last_path = "decode_stream_paged";
  return POPE_OK;
}

}  // extern "C"
