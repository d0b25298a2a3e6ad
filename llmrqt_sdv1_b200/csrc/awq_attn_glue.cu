// The two small kernels that sit between the quantized linears of a decoder layer at decode time (one token):
//
//   qk_norm_rope_cache   the fused-qkv output row -> per-head RMSNorm of q and k (models that have it), rotary
//                        embedding of q and k at the current position, q to a buffer, k and v into the KV cache
//                        (the reference's attention block does these as separate tensor operations:
//                        LLMQRT/runtime_refact/nn_models/modules/nonlinear/attention.py:299-330)
//   attn_decode          one query token against the cached keys / values 0..pos (grouped-query attention),
//                        online softmax in fp32
//
// Both read the position from DEVICE memory, so a decode step that uses them is the same sequence of launches
// for every token and can be captured once in a CUDA graph.  They are the plumbing around the linears, not the
// hot path: written for few launches, not tuned further.  Each fp16 step rounds where the separate fp16 tensor
// operations round (normalised value, times weight, x*cos, rot*sin, their sum).
#include "awq_common.cuh"

namespace awq {

// One warp per head of the qkv row: heads [0, H) are q, [H, H+KV) are k, [H+KV, H+2KV) are v.  D = 32 * V.
template <int V>
__global__ void __launch_bounds__(128)
qk_norm_rope_cache_kernel(const __half* __restrict__ qkv, const __half* __restrict__ q_weight,
                          const __half* __restrict__ k_weight, float eps, const __half* __restrict__ cos_tab,
                          const __half* __restrict__ sin_tab, const long long* __restrict__ pos_ptr,
                          __half* __restrict__ q_out, __half* __restrict__ k_cache, __half* __restrict__ v_cache,
                          int H, int KV, int max_len) {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  constexpr int D = 32 * V;
  const int head = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (head >= H + 2 * KV) return;
  const long long pos = *pos_ptr;
  if (pos < 0 || pos >= max_len) return;              // out of range: leave everything untouched
  const __half* src = qkv + static_cast<size_t>(head) * D + lane * V;
  __half x[V];
#pragma unroll
  for (int i = 0; i < V; ++i) x[i] = src[i];
  if (head >= H + KV) {                               // v: straight into the cache
    __half* dst = v_cache + (static_cast<size_t>(head - H - KV) * max_len + pos) * D + lane * V;
#pragma unroll
    for (int i = 0; i < V; ++i) dst[i] = x[i];
    return;
  }
  const bool is_q = head < H;
  const __half* w = is_q ? q_weight : k_weight;
  if (w != nullptr) {
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < V; ++i) { const float f = __half2float(x[i]); ss = fmaf(f, f, ss); }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    const float r = rsqrtf(ss / D + eps);
#pragma unroll
    for (int i = 0; i < V; ++i)
      x[i] = __hmul_rn(w[lane * V + i], __float2half_rn(__half2float(x[i]) * r));
  }
  // rotate_half: element i pairs with i + D/2 (first half, negated partner) or i - D/2 (second half): lane ^ 16
  const __half* cs = cos_tab + static_cast<size_t>(pos) * D + lane * V;
  const __half* sn = sin_tab + static_cast<size_t>(pos) * D + lane * V;
  __half out[V];
#pragma unroll
  for (int i = 0; i < V; ++i) {
    const unsigned partner = __shfl_xor_sync(0xffffffffu, static_cast<unsigned>(__half_as_ushort(x[i])), 16);
    __half rot = __ushort_as_half(static_cast<unsigned short>(partner));
    if (lane < 16) rot = __hneg(rot);
    out[i] = __hadd_rn(__hmul_rn(x[i], cs[i]), __hmul_rn(rot, sn[i]));    // three roundings, never contracted
  }
  __half* dst = is_q ? q_out + static_cast<size_t>(head) * D + lane * V
                     : k_cache + (static_cast<size_t>(head - H) * max_len + pos) * D + lane * V;
#pragma unroll
  for (int i = 0; i < V; ++i) dst[i] = out[i];
}

// One CTA per query head; its 16 warps take the cached positions in turn, four at a time (the eight loads of a
// batch - four key rows, four value rows - are issued together: a lone dependent load per position would make the
// kernel pay one memory latency per cached token).  Lane = V of the D dimensions.  Every warp keeps its own
// running maximum / sum / weighted values; they are merged through shared memory at the end.
constexpr int kAttnWarps = 16;
constexpr int kAttnBatch = 4;

template <int V>
__device__ __forceinline__ void load_row(const __half* p, float (&f)[V]) {
  if constexpr (V == 4) {
    const uint2 u = __ldg(reinterpret_cast<const uint2*>(p));
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&u.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
  } else {
    const uint32_t u = __ldg(reinterpret_cast<const uint32_t*>(p));
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&u));
    f[0] = a.x; f[1] = a.y;
  }
}

template <int V>
__global__ void __launch_bounds__(kAttnWarps * 32)
attn_decode_kernel(const __half* __restrict__ q, const __half* __restrict__ k_cache, const __half* __restrict__ v_cache,
                   const long long* __restrict__ pos_ptr, __half* __restrict__ out, int H, int KV, int max_len,
                   float scale) {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  static_assert(V == 2 || V == 4, "head dimension 64 or 128");
  constexpr int D = 32 * V;
  constexpr int W = kAttnWarps, B = kAttnBatch;
  __shared__ float s_m[W], s_l[W], s_acc[W][D];
  const int head = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kv = head / (H / KV);
  long long pos = *pos_ptr;
  if (pos >= max_len) pos = max_len - 1;
  float qf[V];
#pragma unroll
  for (int i = 0; i < V; ++i) qf[i] = __half2float(q[static_cast<size_t>(head) * D + lane * V + i]) * scale;
  const __half* kb = k_cache + static_cast<size_t>(kv) * max_len * D + lane * V;
  const __half* vb = v_cache + static_cast<size_t>(kv) * max_len * D + lane * V;
  float m = -INFINITY, l = 0.f, acc[V];
#pragma unroll
  for (int i = 0; i < V; ++i) acc[i] = 0.f;
  for (long long j0 = static_cast<long long>(warp) * B; j0 <= pos; j0 += W * B) {
    float kf[B][V], vf[B][V];
#pragma unroll
    for (int b = 0; b < B; ++b) {
      const long long j = (j0 + b <= pos) ? j0 + b : pos;        // a repeated row past the end; masked out below
      load_row<V>(kb + j * D, kf[b]);
      load_row<V>(vb + j * D, vf[b]);
    }
    float s[B];
#pragma unroll
    for (int b = 0; b < B; ++b) {
      s[b] = 0.f;
#pragma unroll
      for (int i = 0; i < V; ++i) s[b] = fmaf(qf[i], kf[b][i], s[b]);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
      for (int b = 0; b < B; ++b) s[b] += __shfl_xor_sync(0xffffffffu, s[b], off);
    }
    float m_new = m;
#pragma unroll
    for (int b = 0; b < B; ++b) {
      if (j0 + b > pos) s[b] = -INFINITY;
      m_new = fmaxf(m_new, s[b]);
    }
    const float corr = __expf(m - m_new);                        // m_new is finite: position j0 is valid
    l *= corr;
#pragma unroll
    for (int i = 0; i < V; ++i) acc[i] *= corr;
#pragma unroll
    for (int b = 0; b < B; ++b) {
      const float pj = __expf(s[b] - m_new);                     // 0 for masked positions
      l += pj;
#pragma unroll
      for (int i = 0; i < V; ++i) acc[i] = fmaf(pj, vf[b][i], acc[i]);
    }
    m = m_new;
  }
  if (lane == 0) { s_m[warp] = m; s_l[warp] = l; }
#pragma unroll
  for (int i = 0; i < V; ++i) s_acc[warp][lane * V + i] = acc[i];
  __syncthreads();
  if (warp == 0) {
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < W; ++w) M = fmaxf(M, s_m[w]);
    float L = 0.f, o[V];
#pragma unroll
    for (int i = 0; i < V; ++i) o[i] = 0.f;
#pragma unroll
    for (int w = 0; w < W; ++w) {
      const float c = (s_m[w] == -INFINITY) ? 0.f : __expf(s_m[w] - M);
      L = fmaf(s_l[w], c, L);
#pragma unroll
      for (int i = 0; i < V; ++i) o[i] = fmaf(s_acc[w][lane * V + i], c, o[i]);
    }
    const float inv = L > 0.f ? 1.f / L : 0.f;
#pragma unroll
    for (int i = 0; i < V; ++i) out[static_cast<size_t>(head) * D + lane * V + i] = __float2half_rn(o[i] * inv);
  }
}

template <typename... Args>
static int launch_pdl(void (*kernel)(Args...), dim3 grid, dim3 block, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  AWQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, args...));
  return AWQ_B200_OK;
}

}  // namespace awq

extern "C" {

int awq_b200_qk_norm_rope_cache(const void* qkv, const void* q_weight, const void* k_weight, float eps,
                                const void* cos_tab, const void* sin_tab, const int64_t* pos, void* q_out,
                                void* k_cache, void* v_cache, int H, int KV, int D, int max_len,
                                awq_b200_stream_t stream) {
  using namespace awq;
  if (!qkv || !cos_tab || !sin_tab || !pos || !q_out || !k_cache || !v_cache) return AWQ_B200_ERR_NULL;
  if ((q_weight == nullptr) != (k_weight == nullptr)) return AWQ_B200_ERR_NULL;
  if (H < 1 || KV < 1 || H % KV != 0 || max_len < 1 || (D != 64 && D != 128)) return AWQ_B200_ERR_SHAPE;
  const int heads = H + 2 * KV;
  const dim3 grid((heads + 3) / 4), block(128);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const __half* a = static_cast<const __half*>(qkv);
  const __half *qw = static_cast<const __half*>(q_weight), *kw = static_cast<const __half*>(k_weight);
  const __half *ct = static_cast<const __half*>(cos_tab), *st = static_cast<const __half*>(sin_tab);
  const long long* pp = reinterpret_cast<const long long*>(pos);
  __half *qo = static_cast<__half*>(q_out), *kc = static_cast<__half*>(k_cache), *vc = static_cast<__half*>(v_cache);
  if (D == 128) return launch_pdl(qk_norm_rope_cache_kernel<4>, grid, block, s, a, qw, kw, eps, ct, st, pp, qo, kc, vc, H, KV, max_len);
  return launch_pdl(qk_norm_rope_cache_kernel<2>, grid, block, s, a, qw, kw, eps, ct, st, pp, qo, kc, vc, H, KV, max_len);
}

int awq_b200_attn_decode(const void* q, const void* k_cache, const void* v_cache, const int64_t* pos, void* out, int H,
                         int KV, int D, int max_len, float scale, awq_b200_stream_t stream) {
  using namespace awq;
  if (!q || !k_cache || !v_cache || !pos || !out) return AWQ_B200_ERR_NULL;
  if (H < 1 || KV < 1 || H % KV != 0 || max_len < 1 || (D != 64 && D != 128)) return AWQ_B200_ERR_SHAPE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const __half *qq = static_cast<const __half*>(q), *kc = static_cast<const __half*>(k_cache);
  const __half* vc = static_cast<const __half*>(v_cache);
  const long long* pp = reinterpret_cast<const long long*>(pos);
  __half* o = static_cast<__half*>(out);
  if (D == 128) return launch_pdl(attn_decode_kernel<4>, dim3(H), dim3(kAttnWarps * 32), s, qq, kc, vc, pp, o, H, KV, max_len, scale);
  return launch_pdl(attn_decode_kernel<2>, dim3(H), dim3(kAttnWarps * 32), s, qq, kc, vc, pp, o, H, KV, max_len, scale);
}

}  // extern "C"
