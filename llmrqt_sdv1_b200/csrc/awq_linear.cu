// Row-count dispatch between the decode GEMV and the prefill GEMM.
#include "awq_common.cuh"

namespace {
constexpr size_t kGemmStatusBytes = 256;  // leading slot of the shared workspace: GEMM status word
}

extern "C" {

size_t awq_b200_linear_workspace_bytes(int M, int K, int N) {
  const int gemv_rows = M < awq_b200_gemv_max_rows() ? M : awq_b200_gemv_max_rows();
  return kGemmStatusBytes + awq_b200_gemv_workspace_bytes(gemv_rows < 1 ? 1 : gemv_rows, K, N);
}

// Workspace layout: [0, 256) GEMM status word (zero unless a device-side wait
// expired), then the GEMV workspace (arrival counters first).  All of it must
// be zero before the first call.
int awq_b200_linear_ex(const void* x, const void* packed, const void* scales, const int32_t* qzeros,
                       const void* bias, void* y, int M, int K, int N, int group_size, void* workspace,
                       size_t workspace_bytes, awq_b200_stream_t stream, unsigned flags) {
  if (M < 1) return AWQ_B200_ERR_SHAPE;
  if (!workspace || workspace_bytes < kGemmStatusBytes) return AWQ_B200_ERR_WORKSPACE;
  if (M <= awq_b200_gemv_max_rows()) {
    return awq_b200_gemv_ex(x, packed, scales, qzeros, bias, y, M, K, N, group_size,
                            static_cast<unsigned char*>(workspace) + kGemmStatusBytes,
                            workspace_bytes - kGemmStatusBytes, stream, flags);
  }
  return awq_b200_gemm(x, packed, scales, qzeros, bias, y, M, K, N, group_size, workspace,
                       kGemmStatusBytes, stream);
}

int awq_b200_linear(const void* x, const void* packed, const void* scales, const int32_t* qzeros,
                    const void* bias, void* y, int M, int K, int N, int group_size, void* workspace,
                    size_t workspace_bytes, awq_b200_stream_t stream) {
  return awq_b200_linear_ex(x, packed, scales, qzeros, bias, y, M, K, N, group_size, workspace, workspace_bytes,
                            stream, 0u);
}

}  // extern "C"
