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
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // the next kernel may start its own prefetch
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

// Long contexts: beyond kAttnSplitFrom positions the cached positions of a head are cut into chunks of about
// kAttnChunk positions (whole batches of all warps; longer ones when the launch has too few CTAs per head), one
// CTA per (head, chunk) - gridDim.y CTAs per head are launched, those beyond the chunks of the current position
// leave at once.  A chunk's CTA writes its running maximum, sum and weighted values to the workspace and draws a
// ticket; the CTA that draws the last ticket of its head adds the chunks in chunk order and writes the output
// (deterministic; the counter is left at zero).  Up to kAttnSplitFrom positions there is one chunk, no workspace
// traffic and no ticket: the arithmetic of the unsplit kernel (a ticket costs about what 100 positions do).
constexpr int kAttnSplitFrom = 256;
constexpr int kAttnChunk = 128;
constexpr int kAttnMaxSplits = 8;

struct AttnSplit {
  float* part;          // [H][gridDim.y][2 + D]: maximum, sum, weighted values of a chunk; nullptr: never split
  unsigned* counters;   // [H], zero between launches
};

// Chunk c of n = pos + 1 positions: [lo, hi]; returns the number of chunks (c >= chunks: nothing to do).
__device__ __forceinline__ int attn_chunk(long long n64, int max_splits, int c, long long* lo, long long* hi) {
  constexpr int kStep = kAttnWarps * kAttnBatch;
  const int n = static_cast<int>(n64);                       // n <= max_len, an int
  if (n <= kAttnSplitFrom || max_splits <= 1) {
    *lo = 0;
    *hi = n - 1;
    return 1;
  }
  int chunks = (n + kAttnChunk - 1) / kAttnChunk;
  if (chunks > max_splits) chunks = max_splits;
  int len = (n + chunks - 1) / chunks;
  len = (len + kStep - 1) / kStep * kStep;
  chunks = (n + len - 1) / len;
  *lo = static_cast<long long>(c) * len;
  *hi = (c + 1) * len - 1 < n - 1 ? (c + 1) * len - 1 : n - 1;
  return chunks;
}

// Warp 0 of a chunk's CTA: one chunk -> the output row; several -> the partial, a ticket, and for the last ticket
// of the head the sum over the chunks.
template <int V>
__device__ __forceinline__ void attn_finish(const AttnSplit& sp, int head, int chunk, int chunks, int lane, float M, float L,
                                            const float (&o)[V], __half* __restrict__ out) {
  constexpr int D = 32 * V;
  if (chunks == 1) {
    const float inv = L > 0.f ? 1.f / L : 0.f;
#pragma unroll
    for (int i = 0; i < V; ++i) out[static_cast<size_t>(head) * D + lane * V + i] = __float2half_rn(o[i] * inv);
    return;
  }
  const int S = static_cast<int>(gridDim.y);
  float* mine = sp.part + (static_cast<size_t>(head) * S + chunk) * (D + 2);
  if (lane == 0) { __stcg(mine, M); __stcg(mine + 1, L); }
#pragma unroll
  for (int i = 0; i < V; ++i) __stcg(mine + 2 + lane * V + i, o[i]);
  __threadfence();
  __syncwarp();
  unsigned ticket = 0u;
  if (lane == 0) ticket = atomicAdd(sp.counters + head, 1u);
  ticket = __shfl_sync(0xffffffffu, ticket, 0);
  if (ticket != static_cast<unsigned>(chunks - 1)) return;
  __threadfence();
  // Eight chunks at a time: their loads first (one memory latency for the lot), then the sums in chunk order
  // under a running maximum.
  const float* base = sp.part + static_cast<size_t>(head) * S * (D + 2);
  constexpr int kGroup = 8;
  float Mt = -INFINITY, Lt = 0.f, ot[V];
#pragma unroll
  for (int i = 0; i < V; ++i) ot[i] = 0.f;
  for (int c0 = 0; c0 < chunks; c0 += kGroup) {
    float Mc[kGroup], Lc[kGroup], oc[kGroup][V];
#pragma unroll
    for (int c = 0; c < kGroup; ++c) {
      const float* pc = base + static_cast<size_t>(c0 + c < chunks ? c0 + c : c0) * (D + 2);
      Mc[c] = __ldcg(pc);
      Lc[c] = __ldcg(pc + 1);
#pragma unroll
      for (int i = 0; i < V; ++i) oc[c][i] = __ldcg(pc + 2 + lane * V + i);
    }
    float Mn = Mt;
#pragma unroll
    for (int c = 0; c < kGroup; ++c)
      if (c0 + c < chunks) Mn = fmaxf(Mn, Mc[c]);
    const float corr = __expf(Mt - Mn);                            // Mn is finite: every chunk holds a position
    Lt *= corr;
#pragma unroll
    for (int i = 0; i < V; ++i) ot[i] *= corr;
#pragma unroll
    for (int c = 0; c < kGroup; ++c) {
      if (c0 + c < chunks) {                                       // warp-uniform
        const float f = __expf(Mc[c] - Mn);
        Lt = fmaf(Lc[c], f, Lt);
#pragma unroll
        for (int i = 0; i < V; ++i) ot[i] = fmaf(oc[c][i], f, ot[i]);
      }
    }
    Mt = Mn;
  }
  const float inv = Lt > 0.f ? 1.f / Lt : 0.f;
#pragma unroll
  for (int i = 0; i < V; ++i) out[static_cast<size_t>(head) * D + lane * V + i] = __float2half_rn(ot[i] * inv);
  if (lane == 0) sp.counters[head] = 0u;     // every chunk has drawn its ticket: leave the counter clean
}

template <int V>
__global__ void __launch_bounds__(kAttnWarps * 32)
attn_decode_kernel(const __half* __restrict__ q, const __half* __restrict__ k_cache, const __half* __restrict__ v_cache,
                   const long long* __restrict__ pos_ptr, __half* __restrict__ out, int H, int KV, int max_len,
                   float scale, AttnSplit sp) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // the next kernel may start its own prefetch
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
  if (pos < 0) pos = 0;
  long long lo, hi;
  const int chunks = attn_chunk(pos + 1, static_cast<int>(gridDim.y), static_cast<int>(blockIdx.y), &lo, &hi);
  if (static_cast<int>(blockIdx.y) >= chunks) return;              // CTA-uniform
  float qf[V];
#pragma unroll
  for (int i = 0; i < V; ++i) qf[i] = __half2float(q[static_cast<size_t>(head) * D + lane * V + i]) * scale;
  const __half* kb = k_cache + static_cast<size_t>(kv) * max_len * D + lane * V;
  const __half* vb = v_cache + static_cast<size_t>(kv) * max_len * D + lane * V;
  float m = -INFINITY, l = 0.f, acc[V];
#pragma unroll
  for (int i = 0; i < V; ++i) acc[i] = 0.f;
  if (chunks == 1) {
    // The whole context in this CTA (always so up to kAttnSplitFrom positions).  The loop is written out a
    // second time with the chunk's bounds below: with lo / hi as its bounds the compiler schedules this loop
    // worse (one CTA per head: 26 instead of 17 us at 1000 positions), and short contexts are the common case.
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
  } else {
    for (long long j0 = lo + static_cast<long long>(warp) * B; j0 <= hi; j0 += W * B) {
      float kf[B][V], vf[B][V];
#pragma unroll
      for (int b = 0; b < B; ++b) {
        const long long j = (j0 + b <= hi) ? j0 + b : hi;        // a repeated row past the end; masked out below
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
        if (j0 + b > hi) s[b] = -INFINITY;
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
    attn_finish<V>(sp, head, static_cast<int>(blockIdx.y), chunks, lane, M, L, o, out);
  }
}

// The two kernels above as ONE launch per layer: CTA h first turns its own query head and the key / value head of its
// group into their final fp16 values (warps 0, 1, 2: per-head RMSNorm, rotary embedding - the arithmetic of
// qk_norm_rope_cache_kernel), keeps them in shared memory, and then attends over the cached positions 0..pos-1 plus
// the fresh key / value.  The first CTA of a group also writes the fresh key / value into row `pos` of the cache for
// the tokens to come; no CTA reads that row in this launch, so CTAs never wait for one another.  Same bits as the
// two-kernel sequence (the positions are visited in the same batches).
template <int V>
__device__ __forceinline__ void norm_rope_head(const __half* __restrict__ src, const __half* __restrict__ w, float eps,
                                               const __half* __restrict__ cs, const __half* __restrict__ sn, bool rope,
                                               int lane, __half (&out)[V]) {
  constexpr int D = 32 * V;
  __half x[V];
#pragma unroll
  for (int i = 0; i < V; ++i) x[i] = src[lane * V + i];
  if (w != nullptr) {
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < V; ++i) { const float f = __half2float(x[i]); ss = fmaf(f, f, ss); }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    const float r = rsqrtf(ss / D + eps);
#pragma unroll
    for (int i = 0; i < V; ++i) x[i] = __hmul_rn(w[lane * V + i], __float2half_rn(__half2float(x[i]) * r));
  }
#pragma unroll
  for (int i = 0; i < V; ++i) {
    if (rope) {
      const unsigned partner = __shfl_xor_sync(0xffffffffu, static_cast<unsigned>(__half_as_ushort(x[i])), 16);
      __half rot = __ushort_as_half(static_cast<unsigned short>(partner));
      if (lane < 16) rot = __hneg(rot);
      out[i] = __hadd_rn(__hmul_rn(x[i], cs[lane * V + i]), __hmul_rn(rot, sn[lane * V + i]));
    } else {
      out[i] = x[i];
    }
  }
}

template <int V>
__global__ void __launch_bounds__(kAttnWarps * 32)
attn_step_kernel(const __half* __restrict__ qkv, const __half* __restrict__ q_weight, const __half* __restrict__ k_weight,
                 float eps, const __half* __restrict__ cos_tab, const __half* __restrict__ sin_tab,
                 const long long* __restrict__ pos_ptr, __half* __restrict__ k_cache, __half* __restrict__ v_cache,
                 __half* __restrict__ out, int H, int KV, int max_len, float scale, AttnSplit sp) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // the next kernel may start its own prefetch
  asm volatile("griddepcontrol.wait;" ::: "memory");
  static_assert(V == 2 || V == 4, "head dimension 64 or 128");
  constexpr int D = 32 * V;
  constexpr int W = kAttnWarps, B = kAttnBatch;
  __shared__ float s_m[W], s_l[W], s_acc[W][D];
  __shared__ __half s_q[D], s_k[D], s_v[D];
  const int head = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = H / KV;
  const int kv = head / group;
  const long long pos = *pos_ptr;
  if (pos < 0 || pos >= max_len) return;              // out of range: leave everything untouched (CTA-uniform)
  long long lo, hi;
  const int chunks = attn_chunk(pos + 1, static_cast<int>(gridDim.y), static_cast<int>(blockIdx.y), &lo, &hi);
  if (static_cast<int>(blockIdx.y) >= chunks) return;              // CTA-uniform
  if (warp < 3) {
    const __half* cs = cos_tab + static_cast<size_t>(pos) * D;
    const __half* sn = sin_tab + static_cast<size_t>(pos) * D;
    __half o[V];
    if (warp == 0) {
      norm_rope_head<V>(qkv + static_cast<size_t>(head) * D, q_weight, eps, cs, sn, true, lane, o);
#pragma unroll
      for (int i = 0; i < V; ++i) s_q[lane * V + i] = o[i];
    } else {
      const bool is_k = warp == 1;
      norm_rope_head<V>(qkv + static_cast<size_t>(is_k ? H + kv : H + KV + kv) * D, is_k ? k_weight : nullptr, eps, cs, sn,
                        is_k, lane, o);
      __half* keep = is_k ? s_k : s_v;
#pragma unroll
      for (int i = 0; i < V; ++i) keep[lane * V + i] = o[i];
      if (head == kv * group && blockIdx.y == 0) {       // one CTA per group appends to the cache
        __half* dst = (is_k ? k_cache : v_cache) + (static_cast<size_t>(kv) * max_len + pos) * D + lane * V;
#pragma unroll
        for (int i = 0; i < V; ++i) dst[i] = o[i];
      }
    }
  }
  __syncthreads();
  float qf[V], knew[V], vnew[V];
#pragma unroll
  for (int i = 0; i < V; ++i) {
    qf[i] = __half2float(s_q[lane * V + i]) * scale;
    knew[i] = __half2float(s_k[lane * V + i]);
    vnew[i] = __half2float(s_v[lane * V + i]);
  }
  const __half* kb = k_cache + static_cast<size_t>(kv) * max_len * D + lane * V;
  const __half* vb = v_cache + static_cast<size_t>(kv) * max_len * D + lane * V;
  float m = -INFINITY, l = 0.f, acc[V];
#pragma unroll
  for (int i = 0; i < V; ++i) acc[i] = 0.f;
  if (chunks == 1) {
    // The whole context in this CTA (always so up to kAttnSplitFrom positions).  The loop is written out a
    // second time with the chunk's bounds below: with lo / hi as its bounds the compiler schedules this loop
    // worse (one CTA per head: 26 instead of 17 us at 1000 positions), and short contexts are the common case.
    for (long long j0 = static_cast<long long>(warp) * B; j0 <= pos; j0 += W * B) {
      float kf[B][V], vf[B][V];
#pragma unroll
      for (int b = 0; b < B; ++b) {
        const long long j = j0 + b;
        if (j < pos) {                                              // warp-uniform
          load_row<V>(kb + j * D, kf[b]);
          load_row<V>(vb + j * D, vf[b]);
        } else {                                                    // the fresh row (and the masked slots behind it)
#pragma unroll
          for (int i = 0; i < V; ++i) { kf[b][i] = knew[i]; vf[b][i] = vnew[i]; }
        }
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
  } else {
    for (long long j0 = lo + static_cast<long long>(warp) * B; j0 <= hi; j0 += W * B) {
      float kf[B][V], vf[B][V];
#pragma unroll
      for (int b = 0; b < B; ++b) {
        const long long j = j0 + b;
        if (j < pos) {                                              // warp-uniform
          load_row<V>(kb + j * D, kf[b]);
          load_row<V>(vb + j * D, vf[b]);
        } else {                                                    // the fresh row (and the masked slots behind it)
#pragma unroll
          for (int i = 0; i < V; ++i) { kf[b][i] = knew[i]; vf[b][i] = vnew[i]; }
        }
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
        if (j0 + b > hi) s[b] = -INFINITY;
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
    attn_finish<V>(sp, head, static_cast<int>(blockIdx.y), chunks, lane, M, L, o, out);
  }
}

// RMSNorm of M rows of width D (fp16 in, fp16 weight, fp16 out): y = fp16( (x * rsqrt(mean(x^2) + eps)) * w ), all
// in fp32 with ONE rounding at the end, as torch.nn.functional.rms_norm computes it (the reference's decoder layers
// call their norm modules between the linears: LLMQRT/runtime_refact/nn_models/modules/nonlinear/
// transformer_layer.py:139-151).  One CTA per row; a launch that can overlap its predecessor's tail.
constexpr int kNormThreads = 256;
constexpr int kNormKeep = 8;          // pairs a thread keeps in registers between the two passes (rows up to 4096 wide)
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_kernel(const __half* __restrict__ x, const __half* __restrict__ w, float eps, __half* __restrict__ y, int D) {
  // the weight is constant data: fetch it while the predecessor still runs
  const int pairs = D >> 1;
  float2 g[kNormKeep];
#pragma unroll
  for (int j = 0; j < kNormKeep; ++j) {
    const int i = threadIdx.x + j * kNormThreads;
    g[j] = make_float2(0.f, 0.f);
    if (i < pairs) g[j] = __half22float2(*reinterpret_cast<const __half2*>(w + 2 * i));
  }
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // the next kernel may start its own prefetch
  asm volatile("griddepcontrol.wait;" ::: "memory");
  __shared__ float red[kNormThreads / 32];
  const __half* xr = x + static_cast<size_t>(blockIdx.x) * D;
  __half* yr = y + static_cast<size_t>(blockIdx.x) * D;
  float2 f[kNormKeep];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < kNormKeep; ++j) {
    const int i = threadIdx.x + j * kNormThreads;
    f[j] = make_float2(0.f, 0.f);
    if (i < pairs) f[j] = __half22float2(*reinterpret_cast<const __half2*>(xr + 2 * i));
  }
#pragma unroll
  for (int j = 0; j < kNormKeep; ++j) {            // fixed order of additions, whatever the row's width
    ss = fmaf(f[j].x, f[j].x, ss);
    ss = fmaf(f[j].y, f[j].y, ss);
  }
  for (int i = threadIdx.x + kNormKeep * kNormThreads; i < pairs; i += kNormThreads) {
    const float2 v = __half22float2(*reinterpret_cast<const __half2*>(xr + 2 * i));
    ss = fmaf(v.x, v.x, ss);
    ss = fmaf(v.y, v.y, ss);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < kNormThreads / 32; ++i) tot += red[i];
  const float r = rsqrtf(tot / D + eps);
#pragma unroll
  for (int j = 0; j < kNormKeep; ++j) {
    const int i = threadIdx.x + j * kNormThreads;
    if (i < pairs) *reinterpret_cast<__half2*>(yr + 2 * i) = __floats2half2_rn((f[j].x * r) * g[j].x, (f[j].y * r) * g[j].y);
  }
  for (int i = threadIdx.x + kNormKeep * kNormThreads; i < pairs; i += kNormThreads) {
    const float2 v = __half22float2(*reinterpret_cast<const __half2*>(xr + 2 * i));
    const float2 gw = __half22float2(*reinterpret_cast<const __half2*>(w + 2 * i));
    *reinterpret_cast<__half2*>(yr + 2 * i) = __floats2half2_rn((v.x * r) * gw.x, (v.y * r) * gw.y);
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

// Workspace of the attention kernels: [0, 256 * ceil(H / 64)) arrival counters (zero before the first use, left
// zero), then the chunks' partial results.  CTAs per head: what one wave of one 512-thread CTA per SM holds (their
// registers allow one per SM; with two, capped at 64 registers, the position loop ran 15-40 % slower), at most 8.
static int attn_splits(int H) {
  int s = 148 / H;
  if (s < 1) s = 1;
  if (s > kAttnMaxSplits) s = kAttnMaxSplits;
  return s;
}
static size_t attn_counter_bytes(int H) { return (static_cast<size_t>(H) * sizeof(unsigned) + 255) / 256 * 256; }
static size_t attn_workspace_bytes(int H, int D) {
  return attn_counter_bytes(H) + static_cast<size_t>(H) * attn_splits(H) * (D + 2) * sizeof(float);
}
// The split a launch uses: none without a workspace of that size.
static int attn_split_of(void* workspace, size_t workspace_bytes, int H, int D, AttnSplit* sp) {
  sp->part = nullptr;
  sp->counters = nullptr;
  if (workspace == nullptr || workspace_bytes < attn_workspace_bytes(H, D)) return 1;
  sp->counters = static_cast<unsigned*>(workspace);
  sp->part = reinterpret_cast<float*>(static_cast<unsigned char*>(workspace) + attn_counter_bytes(H));
  return attn_splits(H);
}

}  // namespace awq

extern "C" {

size_t awq_b200_attn_workspace_bytes(int H, int D) {
  if (H < 1 || (D != 64 && D != 128)) return 0;
  return awq::attn_workspace_bytes(H, D);
}

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
                         int KV, int D, int max_len, float scale, void* workspace, size_t workspace_bytes,
                         awq_b200_stream_t stream) {
  using namespace awq;
  if (!q || !k_cache || !v_cache || !pos || !out) return AWQ_B200_ERR_NULL;
  if (H < 1 || KV < 1 || H % KV != 0 || max_len < 1 || (D != 64 && D != 128)) return AWQ_B200_ERR_SHAPE;
  if (workspace != nullptr && (reinterpret_cast<uintptr_t>(workspace) & 15u)) return AWQ_B200_ERR_ALIGN;
  AttnSplit sp;
  const dim3 grid(H, attn_split_of(workspace, workspace_bytes, H, D, &sp));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const __half *qq = static_cast<const __half*>(q), *kc = static_cast<const __half*>(k_cache);
  const __half* vc = static_cast<const __half*>(v_cache);
  const long long* pp = reinterpret_cast<const long long*>(pos);
  __half* o = static_cast<__half*>(out);
  if (D == 128) return launch_pdl(attn_decode_kernel<4>, grid, dim3(kAttnWarps * 32), s, qq, kc, vc, pp, o, H, KV, max_len, scale, sp);
  return launch_pdl(attn_decode_kernel<2>, grid, dim3(kAttnWarps * 32), s, qq, kc, vc, pp, o, H, KV, max_len, scale, sp);
}

int awq_b200_attn_step(const void* qkv, const void* q_weight, const void* k_weight, float eps, const void* cos_tab,
                       const void* sin_tab, const int64_t* pos, void* k_cache, void* v_cache, void* out, int H, int KV,
                       int D, int max_len, float scale, void* workspace, size_t workspace_bytes,
                       awq_b200_stream_t stream) {
  using namespace awq;
  if (!qkv || !cos_tab || !sin_tab || !pos || !k_cache || !v_cache || !out) return AWQ_B200_ERR_NULL;
  if ((q_weight == nullptr) != (k_weight == nullptr)) return AWQ_B200_ERR_NULL;
  if (H < 1 || KV < 1 || H % KV != 0 || max_len < 1 || (D != 64 && D != 128)) return AWQ_B200_ERR_SHAPE;
  if (workspace != nullptr && (reinterpret_cast<uintptr_t>(workspace) & 15u)) return AWQ_B200_ERR_ALIGN;
  AttnSplit sp;
  const dim3 grid(H, attn_split_of(workspace, workspace_bytes, H, D, &sp));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const __half* a = static_cast<const __half*>(qkv);
  const __half *qw = static_cast<const __half*>(q_weight), *kw = static_cast<const __half*>(k_weight);
  const __half *ct = static_cast<const __half*>(cos_tab), *st = static_cast<const __half*>(sin_tab);
  const long long* pp = reinterpret_cast<const long long*>(pos);
  __half *kc = static_cast<__half*>(k_cache), *vc = static_cast<__half*>(v_cache), *o = static_cast<__half*>(out);
  if (D == 128) return launch_pdl(attn_step_kernel<4>, grid, dim3(kAttnWarps * 32), s, a, qw, kw, eps, ct, st, pp, kc, vc, o, H, KV, max_len, scale, sp);
  return launch_pdl(attn_step_kernel<2>, grid, dim3(kAttnWarps * 32), s, a, qw, kw, eps, ct, st, pp, kc, vc, o, H, KV, max_len, scale, sp);
}

int awq_b200_rmsnorm(const void* x, const void* weight, float eps, void* y, int M, int D, awq_b200_stream_t stream) {
  using namespace awq;
  if (!x || !weight || !y) return AWQ_B200_ERR_NULL;
  if (M < 1 || D < 2 || (D & 1)) return AWQ_B200_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(y)) & 3u)
    return AWQ_B200_ERR_ALIGN;
  return launch_pdl(rmsnorm_kernel, dim3(M), dim3(kNormThreads), static_cast<cudaStream_t>(stream),
                    static_cast<const __half*>(x), static_cast<const __half*>(weight), eps, static_cast<__half*>(y), D);
}

}  // extern "C"
