// Row-count and shape dispatch between the linear kernels: the mma.sync decode GEMV, the two tensor-memory
// split-K kernels for few rows of a large matrix (integer path up to 8 rows, exact fp16 weights up to 64),
// and the prefill GEMM.
#include "awq_common.cuh"

namespace {
constexpr size_t kGemmStatusBytes = 256;  // leading slot of the shared workspace: GEMM status word
constexpr int kSkinnyMaxRows = 64;

// Which kernel serves M rows of a K x N linear (all thresholds are on (K, N) only, so within a row-count class
// a row's bits do not change with the number of rows decoded together).
//   rows <= 4:  the GEMV, or from 24 MiB of packed weights the integer tensor-core decode kernel
//               (awq_decode_i8.cu; 70B-class gate_up at one row: 45 us against 72 us).
//   5..8:       the GEMV, or from 48 MiB the integer kernel again (its 8-row form).
//   9..16:      the GEMV, or from 16 MiB the exact-weight split-K tensor-memory kernel (beyond 8 rows the GEMV
//               does its unpacking twice).
//   17..64:     small matrices (packed MiB x ceil(rows / 8) <= 32): the GEMV, 8 rows per CTA; else the exact-weight
//               tensor-memory kernel where the GEMM would leave most SMs idle (at most 74 column tiles of 256)
//               and k is long enough to split (at least 32 blocks of 128); the GEMM otherwise.
// Like the reference's own switch from its GEMV to its GEMM at 8 rows (linear_awq.py:167-185), a switch of
// kernel changes the order of additions.
enum class Route { kGemv, kDecodeI8, kSkinny, kGemm };
constexpr int kDecodeI8MaxRows = 4;
Route route(int M, int K, int N, int group_size, bool one_kernel_below_8 = false) {
  // Groups of 32 or 64: only the kernels that build the exact fp16 weight per element take them.
  if (group_size < 128) return M <= kSkinnyMaxRows ? Route::kSkinny : Route::kGemm;
  const long long packed_bytes = static_cast<long long>(K) * N / 2;
  if (one_kernel_below_8 && M < 8) return Route::kGemv;
  if (M <= 16) {
    // Measured crossovers against the GEMV (us, graph replay, weights from HBM): the integer kernel wins from
    // ~16-20 MiB at one row (28 MiB: 10.8-11.2 against 12.5-12.9) and from ~36 MiB at four rows.  One threshold
    // for the class: decode (1 row) and a short verification (2..4 rows) must take the same kernel.
    if (M <= kDecodeI8MaxRows) return packed_bytes < (24ll << 20) ? Route::kGemv : Route::kDecodeI8;
    // 5..8 rows: the integer kernel behind its planes' kernel (70B gate_up 58 us against 75 us of the exact-weight
    // kernel; 56 MiB: 25.3 against 25.8 and 28.5 of the GEMV); the GEMV below 48 MiB (29 MiB: 12.8 against 16.7).
    if (M <= 8) return packed_bytes < (48ll << 20) ? Route::kGemv : Route::kDecodeI8;
    if (packed_bytes < (16ll << 20)) return Route::kGemv;
    return Route::kSkinny;
  }
  // 17..64 rows of a small matrix: the GEMV again, one CTA per 8 rows and column group (the weights are re-read
  // through L2 and unpacked once per 8 rows: ~0.6 us per MiB and 8 rows, against ~20 us of fixed cost in the
  // tensor-memory kernels).  Measured win up to packed MiB x ceil(M / 8) = 32.
  if (M <= kSkinnyMaxRows && packed_bytes * ((M + 7) / 8) <= (32ll << 20)) return Route::kGemv;
  // The split-K kernel's cost grows with the rows, the GEMM's hardly: below 16 MiB the GEMM wins from ~40 rows.
  const bool small_and_many = packed_bytes < (16ll << 20) && M > 32;
  if (M <= kSkinnyMaxRows && !small_and_many && (N + 255) / 256 <= 74 && K / 128 >= 32) return Route::kSkinny;
  return Route::kGemm;
}
}  // namespace

extern "C" {

size_t awq_b200_linear_workspace_bytes(int M, int K, int N) {
  if (M < 1) M = 1;
  // The group size is not known here: take the larger of what the two possible routes of these rows need.
  size_t need = 0;
  switch (route(M, K, N, 128)) {
    case Route::kGemv: need = awq_b200_gemv_workspace_bytes(M, K, N); break;
    case Route::kDecodeI8: need = awq_b200_decode_workspace_bytes(M, K, N); break;
    case Route::kSkinny: need = awq_b200_skinny_workspace_bytes(M, K, N); break;
    case Route::kGemm: return awq_b200_gemm_workspace_bytes(M, K, N);   // status word first there too
  }
  if (M <= kSkinnyMaxRows) {
    const size_t small = awq_b200_skinny_workspace_bytes(M, K, N);
    if (small > need) need = small;
  }
  if (M < 8) {                      // AWQ_B200_ONE_KERNEL_BELOW_8 sends these rows to the GEMV whatever the size
    const size_t gemv = awq_b200_gemv_workspace_bytes(M, K, N);
    if (gemv > need) need = gemv;
  }
  return kGemmStatusBytes + need;
}

// Workspace layout: [0, 256) GEMM status word (zero unless a device-side wait
// expired), then 16 KiB of arrival counters shared by all kernels (each leaves them zero), then
// scratch for partial sums.  The first 256 + 16 KiB bytes must be zero before the first call.
static int linear_run(const void* x, const void* packed, const void* scales, const int32_t* qzeros,
                      const awq::Epilogue& epi, void* y, int M, int K, int N, int group_size, void* workspace,
                      size_t workspace_bytes, awq_b200_stream_t stream, unsigned flags) {
  if (M < 1) return AWQ_B200_ERR_SHAPE;
  if (!workspace || workspace_bytes < kGemmStatusBytes) return AWQ_B200_ERR_WORKSPACE;
  unsigned char* rest = static_cast<unsigned char*>(workspace) + kGemmStatusBytes;
  const size_t rest_bytes = workspace_bytes - kGemmStatusBytes;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (route(M, K, N, group_size, (flags & AWQ_B200_ONE_KERNEL_BELOW_8) != 0)) {
    case Route::kGemv:
      return awq::gemv_run(x, packed, scales, qzeros, epi, y, M, K, N, group_size, rest, rest_bytes, s, flags);
    case Route::kDecodeI8:
      return awq::decode_i8_dispatch(x, packed, scales, qzeros, epi, y, M, K, N, group_size, rest, rest_bytes, s, flags);
    case Route::kSkinny:
      return awq::skinny_dispatch(x, packed, scales, qzeros, epi, y, M, K, N, group_size, rest, rest_bytes, s, flags);
    case Route::kGemm:
      break;
  }
  // Same buffer: the GEMM's counters sit where the decode kernels keep theirs (both leave them zero).
  return awq::gemm_dispatch(x, packed, scales, qzeros, epi, y, M, K, N, group_size, workspace, workspace_bytes, s,
                            (flags & AWQ_B200_GEMM_SMEM) ? 1 : 0);
}

int awq_b200_linear_ex(const void* x, const void* packed, const void* scales, const int32_t* qzeros,
                       const void* bias, void* y, int M, int K, int N, int group_size, void* workspace,
                       size_t workspace_bytes, awq_b200_stream_t stream, unsigned flags) {
  return linear_run(x, packed, scales, qzeros, awq::Epilogue{static_cast<const uint16_t*>(bias), nullptr, 0}, y, M, K,
                    N, group_size, workspace, workspace_bytes, stream, flags);
}

// The linear with the elementwise work that follows it in a decoder layer done in its epilogue: see
// awq_b200_epilogue in the header.  Same routing, workspace and flags as awq_b200_linear_ex.
int awq_b200_linear_fused(const void* x, const void* packed, const void* scales, const int32_t* qzeros,
                          const awq_b200_epilogue* epilogue, void* y, int M, int K, int N, int group_size,
                          void* workspace, size_t workspace_bytes, awq_b200_stream_t stream, unsigned flags) {
  awq::Epilogue epi{nullptr, nullptr, 0};
  if (epilogue != nullptr) {
    if (epilogue->gated != 0 && epilogue->gated != 1) return AWQ_B200_ERR_SHAPE;
    epi.bias = static_cast<const uint16_t*>(epilogue->bias);
    epi.residual = static_cast<const uint16_t*>(epilogue->residual);
    epi.gated = epilogue->gated;
  }
  return linear_run(x, packed, scales, qzeros, epi, y, M, K, N, group_size, workspace, workspace_bytes, stream, flags);
}

int awq_b200_linear(const void* x, const void* packed, const void* scales, const int32_t* qzeros,
                    const void* bias, void* y, int M, int K, int N, int group_size, void* workspace,
                    size_t workspace_bytes, awq_b200_stream_t stream) {
  return awq_b200_linear_ex(x, packed, scales, qzeros, bias, y, M, K, N, group_size, workspace, workspace_bytes,
                            stream, 0u);
}

}  // extern "C"
