// Internal launch entry points shared by the C-ABI dispatcher.  Not part of the public ABI.
#pragma once
#include <cuda_runtime.h>

#include "../../include/pope_b200.h"

namespace pope {

// exact-arithmetic (fp32 FMA) family: any shape / stride / dtype
cudaError_t sim_fwd_simt(const PopeSimArgs& a, cudaStream_t st);
cudaError_t sim_bwd_simt(const PopeSimBwdArgs& a, cudaStream_t st);
size_t attn_fwd_simt_workspace(const PopeAttnArgs& a);
cudaError_t attn_fwd_simt(const PopeAttnArgs& a, cudaStream_t st);
size_t attn_bwd_simt_workspace(const PopeAttnBwdArgs& a);
cudaError_t attn_bwd_simt(const PopeAttnBwdArgs& a, cudaStream_t st);

// tensor-core (tcgen05 + TMEM) family: bf16 / fp16, d in {64, 96, 128}, r % 16 == 0, 2-D freqs
bool attn_fwd_tc_supported(const PopeAttnArgs& a);
size_t attn_fwd_tc_workspace(const PopeAttnArgs& a);
cudaError_t attn_fwd_tc(const PopeAttnArgs& a, cudaStream_t st);
// stand-alone transform q, k -> q', k' (interleaved fp32 layout of the reference) and its backward
cudaError_t apply_qk_fwd(const PopeApplyArgs& a, cudaStream_t st);
cudaError_t apply_qk_bwd(const PopeApplyBwdArgs& a, cudaStream_t st);
// streaming decode (one query row, 16-bit inputs): copy-engine ring + shared-memory transform, HBM-bound
bool decode_stream_supported(const PopeAttnArgs& a);
size_t decode_stream_workspace(const PopeAttnArgs& a);
cudaError_t decode_stream(const PopeAttnArgs& a, cudaStream_t st);
// the same kernel over a paged key / value cache, and the append into the pages
bool decode_paged_supported(const PopePagedDecodeArgs& a);
size_t decode_paged_workspace(const PopePagedDecodeArgs& a);
cudaError_t decode_paged(const PopePagedDecodeArgs& a, cudaStream_t st);
cudaError_t kv_append(const PopeKvAppendArgs& a, cudaStream_t st);
bool sim_fwd_tc_supported(const PopeSimArgs& a);
size_t sim_fwd_tc_workspace(const PopeSimArgs& a);
cudaError_t sim_fwd_tc(const PopeSimArgs& a, cudaStream_t st);
bool sim_bwd_tc_supported(const PopeSimBwdArgs& a);
size_t sim_bwd_tc_workspace(const PopeSimBwdArgs& a);
cudaError_t sim_bwd_tc(const PopeSimBwdArgs& a, cudaStream_t st);
bool attn_bwd_tc_supported(const PopeAttnBwdArgs& a);
size_t attn_bwd_tc_workspace(const PopeAttnBwdArgs& a);
cudaError_t attn_bwd_tc(const PopeAttnBwdArgs& a, cudaStream_t st);
unsigned int tc_read_status();  // sticky device-side status of the tensor-core kernels (synchronises)
cudaError_t tc_clear_status();  // zero that word on the current device (synchronises)
// one CTA that waits on an mbarrier nobody completes, with a tiny try limit: exercises the give-up path of the bounded
// waits (status bit 0 set, TMEM freed, kernel returns) without faulting or hanging the device
cudaError_t tc_selftest_bounded_wait(cudaStream_t st);
void note_last_path(const char* family);  // what pope_b200_last_path() reports on this thread

// delta[b,h,i] = sum_c out[i,c] * dout[i,c]  (fp32, (B,H,Nq) contiguous); used by every backward
cudaError_t attn_bwd_delta(const PopeAttnBwdArgs& a, float* delta, cudaStream_t st);

inline int round_up(int x, int m) { return (x + m - 1) / m * m; }
// 32-wide feature chunks the fp32 attention kernels are instantiated for (d <= 256)
inline int simt_dch(int d) { int c = (d + 31) / 32; return c <= 4 ? c : 8; }

}  // namespace pope
