// Linear attention with a fixed decay per head (a decaying sum of key-value outer products), and
// the kernels around attention mixers whose projections are not grouped per K/V head: the per-head
// norm of queries and keys with the cache write, and the norm-and-gate of a mixer's heads.
//
// Per head, with q_t, k_t [dim] and v_t [v_dim] the activated projections of token t:
//     S_t = decay * S_(t-1) + k_t v_t^T,      o_t = S_t^T q_t,      S = 0 before the first token.
// S [dim, v_dim] lives in float32 in the cache's per-sequence state area, laid out [heads][dim][v_dim],
// and all arithmetic on it is float32 whatever the model dtype.
#include "common.cuh"

namespace {

__device__ __forceinline__ float silu_f(float v) { return v / (1.f + expf(-v)); }
// an activated projection as the model dtype holds it (a bfloat16 model rounds it; float32 keeps it)
template <typename T> __device__ __forceinline__ float act_as(float v, int act_silu) {
  return act_silu ? to_f(from_f<T>(silu_f(v))) : v;
}
__device__ __forceinline__ float sigmoid_f(float v) { return 1.f / (1.f + expf(-v)); }

// ------------------------------------------------------------------------------------------------
// Token by token. One block = one sequence x one head x VB value columns; thread j owns column j of S
// (in shared memory as [dim][VB]) and walks the sequence's new tokens in order.
// proj row t: [q: heads * dim | k: heads * dim | v: heads * v_dim | ...], `stride` elements apart.
template <typename T>
__global__ void linear_attention_scan_kernel(const T* __restrict__ proj, int stride, float* __restrict__ state,
                                             int state_stride, const int* __restrict__ slots, StepBatch sb,
                                             const float* __restrict__ decay, float* __restrict__ out, int heads,
                                             int dim, int v_dim, int act_silu) {
  extern __shared__ float sm[];
  const int VB = blockDim.x;
  float* S = sm;                  // [dim][VB]
  float* qs = S + dim * VB;       // [dim]
  float* ks = qs + dim;           // [dim]
  const int seq = blockIdx.x, h = blockIdx.y, j = blockIdx.z * VB + threadIdx.x;
  const bool mine = j < v_dim;
  const int start = sb.seq_start[seq], n_new = sb.seq_new[seq];
  float* st = state + size_t(slots[seq]) * state_stride + size_t(h) * dim * v_dim;
  const float a = decay[h];
  for (int d = 0; d < dim; ++d) S[d * VB + threadIdx.x] = mine ? st[size_t(d) * v_dim + j] : 0.f;
  const int k_off = heads * dim, v_off = 2 * heads * dim;
  for (int i = 0; i < n_new; ++i) {
    const T* row = proj + size_t(start + i) * stride;
    __syncthreads();    // the previous token's q and k are no longer read
    for (int d = threadIdx.x; d < dim; d += VB) {
      const float qv = to_f(row[h * dim + d]), kv = to_f(row[k_off + h * dim + d]);
      qs[d] = act_as<T>(qv, act_silu);
      ks[d] = act_as<T>(kv, act_silu);
    }
    float v = 0.f;
    if (mine) v = act_as<T>(to_f(row[v_off + h * v_dim + j]), act_silu);
    __syncthreads();
    float o = 0.f;
#pragma unroll 4
    for (int d = 0; d < dim; ++d) {
      const float s = fmaf(a, S[d * VB + threadIdx.x], ks[d] * v);
      S[d * VB + threadIdx.x] = s;
      o = fmaf(s, qs[d], o);
    }
    if (mine) out[(size_t(start + i) * heads + h) * v_dim + j] = o;
  }
  if (mine)
    for (int d = 0; d < dim; ++d) st[size_t(d) * v_dim + j] = S[d * VB + threadIdx.x];
}

// ------------------------------------------------------------------------------------------------
// A step of single tokens: one block = one sequence x one head x a stretch of VJ value columns; the block's threads
// are DS groups of VJ, thread (ds, j) owns rows ds, ds + DS, ... of column j of S, which it reads from the state area,
// updates and writes back (each value is touched once, 32-byte sectors whole); the groups' partial sums
// of o_j meet in shared memory in a fixed order.
template <typename T>
__global__ void __launch_bounds__(512)
linear_attention_token_kernel(const T* __restrict__ proj, int stride, float* __restrict__ state, int state_stride,
                              const int* __restrict__ slots, StepBatch sb, const float* __restrict__ decay,
                              float* __restrict__ out, int heads, int dim, int v_dim, int act_silu, int VJ) {
  extern __shared__ float sm[];
  float* qs = sm;                 // [dim]
  float* ks = qs + dim;           // [dim]
  float* part = ks + dim;         // [DS][VJ]
  const int DS = blockDim.x / VJ;
  const int seq = blockIdx.x, h = blockIdx.y, jj = threadIdx.x % VJ, ds = threadIdx.x / VJ, j = blockIdx.z * VJ + jj;
  const int t = sb.seq_start[seq];
  const T* row = proj + size_t(t) * stride;
  const int k_off = heads * dim, v_off = 2 * heads * dim;
  for (int d = threadIdx.x; d < dim; d += blockDim.x) {
    qs[d] = act_as<T>(to_f(row[h * dim + d]), act_silu);
    ks[d] = act_as<T>(to_f(row[k_off + h * dim + d]), act_silu);
  }
  const bool mine = j < v_dim;
  const float v = mine ? act_as<T>(to_f(row[v_off + h * v_dim + j]), act_silu) : 0.f;
  const float a = decay[h];
  __syncthreads();
  float o = 0.f;
  if (mine) {
    float* col = state + size_t(slots[seq]) * state_stride + size_t(h) * dim * v_dim + j;
    int d = ds;
    for (; d + 3 * DS < dim; d += 4 * DS) {       // four rows in flight
      float s[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) s[u] = col[size_t(d + u * DS) * v_dim];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        s[u] = fmaf(a, s[u], ks[d + u * DS] * v);
        col[size_t(d + u * DS) * v_dim] = s[u];
        o = fmaf(s[u], qs[d + u * DS], o);
      }
    }
    for (; d < dim; d += DS) {
      const float s = fmaf(a, col[size_t(d) * v_dim], ks[d] * v);
      col[size_t(d) * v_dim] = s;
      o = fmaf(s, qs[d], o);
    }
  }
  part[ds * VJ + jj] = o;
  __syncthreads();
  if (ds == 0 && mine) {
    float total = 0.f;
    for (int g = 0; g < DS; ++g) total += part[g * VJ + jj];
    out[(size_t(t) * heads + h) * v_dim + j] = total;
  }
}

// ------------------------------------------------------------------------------------------------
// Chunks of CH tokens, three passes (prompts): with b = decay, a chunk's tokens i = 0..n-1 and S0 the
// state before the chunk,
//     o_i = b^(i+1) S0^T q_i + sum_{s <= i} b^(i-s) (q_i . k_s) v_s,       S_end = b^n S0 + sum_s b^(n-1-s) k_s v_s^T.
// Pass 1 (parallel over chunks): the chunk's own sum  B_c = sum_s b^(n-1-s) k_s v_s^T.
// Pass 2 (per sequence and head, chunks in order): S before every chunk, and the state after the last.
// Pass 3 (parallel over chunks): the outputs. All in float32 on the CUDA cores.
constexpr int CH = 64;

// chunk_seq[c], chunk_q0[c]: sequence and first token (among the sequence's new ones) of chunk c.
// One block = one chunk x one head x VB value columns; thread j owns column j of B (registers over d
// would need dim known; it sits in shared memory).
template <typename T>
__global__ void linear_attention_chunk_sum_kernel(const T* __restrict__ proj, int stride, StepBatch sb,
                                                  const int* __restrict__ chunk_seq, const int* __restrict__ chunk_q0,
                                                  const float* __restrict__ decay, float* __restrict__ sums, int heads,
                                                  int dim, int v_dim, int act_silu) {
  extern __shared__ float sm[];
  const int VB = blockDim.x;
  float* B = sm;                 // [dim][VB]
  float* ks = B + dim * VB;      // [dim]
  const int c = blockIdx.x, h = blockIdx.y, j = blockIdx.z * VB + threadIdx.x;
  const bool mine = j < v_dim;
  const int seq = chunk_seq[c], q0 = chunk_q0[c];
  const int start = sb.seq_start[seq] + q0, n = min(CH, sb.seq_new[seq] - q0);
  const float a = decay[h];
  for (int d = 0; d < dim; ++d) B[d * VB + threadIdx.x] = 0.f;
  const int k_off = heads * dim, v_off = 2 * heads * dim;
  for (int i = 0; i < n; ++i) {
    const T* row = proj + size_t(start + i) * stride;
    __syncthreads();
    for (int d = threadIdx.x; d < dim; d += VB) {
      const float kv = to_f(row[k_off + h * dim + d]);
      ks[d] = act_as<T>(kv, act_silu);
    }
    float v = 0.f;
    if (mine) v = act_as<T>(to_f(row[v_off + h * v_dim + j]), act_silu);
    __syncthreads();
#pragma unroll 4
    for (int d = 0; d < dim; ++d) B[d * VB + threadIdx.x] = fmaf(a, B[d * VB + threadIdx.x], ks[d] * v);
  }
  if (mine) {
    float* dst = sums + (size_t(c) * heads + h) * dim * v_dim;
    for (int d = 0; d < dim; ++d) dst[size_t(d) * v_dim + j] = B[d * VB + threadIdx.x];
  }
}

// One thread per (sequence, head, element of S): walks the sequence's chunks in order; sums[c] becomes the
// state BEFORE chunk c, and the state area receives the state after the last chunk.
__global__ void linear_attention_chunk_join_kernel(float* __restrict__ sums, float* __restrict__ state,
                                                   int state_stride, const int* __restrict__ slots, StepBatch sb,
                                                   const int* __restrict__ seq_chunk0,
                                                   const float* __restrict__ decay, int heads, int dim, int v_dim) {
  const int seq = blockIdx.y;
  const size_t per_head = size_t(dim) * v_dim, per = per_head * heads;
  const size_t e = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (e >= per) return;
  const int h = int(e / per_head);
  const float a = decay[h];
  const int n_new = sb.seq_new[seq], c0 = seq_chunk0[seq];
  float* st = state + size_t(slots[seq]) * state_stride + e;
  float s = *st;
  // a^n by n multiplications: the same product as n single steps would apply; n = CH for all chunks but the last
  float a_full = 1.f, a_last = 1.f;
  const int n_chunks = (n_new + CH - 1) / CH, n_last = n_new - (n_chunks - 1) * CH;
  for (int i = 0; i < CH; ++i) {
    a_full *= a;
    if (i < n_last) a_last *= a;
  }
  constexpr int AHEAD = 8;      // chunks whose own sums are loaded before the chain of updates needs them
  for (int g0 = 0; g0 < n_chunks; g0 += AHEAD) {
    float own[AHEAD];
#pragma unroll
    for (int i = 0; i < AHEAD; ++i) own[i] = (g0 + i < n_chunks) ? sums[size_t(c0 + g0 + i) * per + e] : 0.f;
#pragma unroll
    for (int i = 0; i < AHEAD; ++i) {
      if (g0 + i >= n_chunks) break;
      sums[size_t(c0 + g0 + i) * per + e] = s;
      s = fmaf(g0 + i == n_chunks - 1 ? a_last : a_full, s, own[i]);
    }
  }
  *st = s;
}

// One block = one chunk x one head; 256 threads. Scores of the chunk A[i][s] = b^(i-s) (q_i . k_s) for
// s <= i are formed in shared memory, then o_i = b^(i+1) S0^T q_i + sum_s A[i][s] v_s with thread groups
// over (token, value column).
template <typename T>
__global__ void __launch_bounds__(256)
linear_attention_chunk_out_kernel(const T* __restrict__ proj, int stride, StepBatch sb, const int* __restrict__ chunk_seq,
                                  const int* __restrict__ chunk_q0, const float* __restrict__ decay,
                                  const float* __restrict__ before, float* __restrict__ out, int heads, int dim,
                                  int v_dim, int act_silu) {
  extern __shared__ float sm[];
  float* qs = sm;                       // [CH][dim + 1]
  float* ks = qs + CH * (dim + 1);      // [CH][dim + 1]
  float* A = ks + CH * (dim + 1);       // [CH][CH + 1]
  float* pw = A + CH * (CH + 1);        // [CH + 1]: b^0 .. b^CH
  const int c = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int seq = chunk_seq[c], q0 = chunk_q0[c];
  const int start = sb.seq_start[seq] + q0, n = min(CH, sb.seq_new[seq] - q0);
  const float a = decay[h];
  const int k_off = heads * dim, v_off = 2 * heads * dim;
  if (tid == 0) {
    float p = 1.f;
    for (int i = 0; i <= CH; ++i) {
      pw[i] = p;
      p *= a;
    }
  }
  for (int idx = tid; idx < CH * dim; idx += 256) {
    const int i = idx / dim, d = idx % dim;
    float qv = 0.f, kv = 0.f;
    if (i < n) {
      const T* row = proj + size_t(start + i) * stride;
      qv = act_as<T>(to_f(row[h * dim + d]), act_silu);
      kv = act_as<T>(to_f(row[k_off + h * dim + d]), act_silu);
    }
    qs[i * (dim + 1) + d] = qv;
    ks[i * (dim + 1) + d] = kv;
  }
  __syncthreads();
  for (int idx = tid; idx < CH * CH; idx += 256) {
    const int i = idx / CH, s = idx % CH;
    float dot = 0.f;
    if (s <= i && i < n) {
      const float* qr = qs + i * (dim + 1);
      const float* kr = ks + s * (dim + 1);
      for (int d = 0; d < dim; ++d) dot = fmaf(qr[d], kr[d], dot);
      dot *= pw[i - s];
    }
    A[i * (CH + 1) + s] = dot;
  }
  __syncthreads();
  const float* S0 = before + (size_t(c) * heads + h) * dim * v_dim;
  for (int idx = tid; idx < CH * v_dim; idx += 256) {
    const int i = idx / v_dim, j = idx % v_dim;
    if (i >= n) continue;
    float inter = 0.f;
    const float* qr = qs + i * (dim + 1);
    for (int d = 0; d < dim; ++d) inter = fmaf(S0[size_t(d) * v_dim + j], qr[d], inter);
    float o = inter * pw[i + 1];
    const float* ar = A + i * (CH + 1);
    for (int s = 0; s <= i; ++s) {
      const float v = act_as<T>(to_f(proj[size_t(start + s) * stride + v_off + h * v_dim + j]), act_silu);
      o = fmaf(ar[s], v, o);
    }
    out[(size_t(start + i) * heads + h) * v_dim + j] = o;
  }
}

// ------------------------------------------------------------------------------------------------
// y[t, i] = x[t, i] / sqrt(mean_i x[t, i]^2 + eps) * gain[i] * sigmoid(gate[t, i]) * out_scale: the heads of a
// mixer side by side, normed together and gated. x float32 [n, width]; gate (TG) and y (TO) rows may lie wider apart.
template <typename TG, typename TO>
__global__ void norm_gate_kernel(const float* __restrict__ x, const float* __restrict__ gain, const TG* __restrict__ gate,
                                 int gate_stride, TO* __restrict__ y, int y_stride, int width, float eps,
                                 float out_scale) {
  __shared__ float scratch[32];
  const size_t t = blockIdx.x;
  const float* row = x + t * width;
  float q = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) q = fmaf(row[i], row[i], q);
  const float rstd = 1.0f / sqrtf(block_sum(q, scratch) / float(width) + eps);
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float v = row[i] * rstd * gain[i];
    if (gate) v *= sigmoid_f(to_f(gate[t * gate_stride + i]));
    y[t * y_stride + i] = from_f<TO>(v * out_scale);
  }
}

// ------------------------------------------------------------------------------------------------
// Projection row t: [q: heads * dim | k: kv_heads * dim | v: kv_heads * v_dim | ...] -> queries
// q_out [n_tokens, heads, dim] and the token's K and V rows in the paged pools. With gains, every query
// and key head is divided by its root mean square (eps inside the root) and multiplied by the gain [dim]
// that all heads share; statistics in float32. One block per token, a warp per head.
template <typename T>
__global__ void qk_norm_store_kernel(const T* __restrict__ proj, int stride, T* __restrict__ q_out,
                                     T* __restrict__ k_pool, T* __restrict__ v_pool, StepBatch sb,
                                     const float* __restrict__ q_gain, const float* __restrict__ k_gain, int heads,
                                     int kv_heads, int dim, int v_dim, float eps, int write_cache) {
  const int t = blockIdx.x;
  const int pos = sb.tok_pos[t], seq = sb.tok_seq[t];
  const int page = sb.pages[size_t(seq) * sb.pages_stride + pos / PTB_PAGE], in_page = pos % PTB_PAGE;
  const T* row = proj + size_t(t) * stride;
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32, n_warps = blockDim.x / 32;
  for (int hh = warp; hh < heads + kv_heads; hh += n_warps) {
    const bool is_q = hh < heads;
    if (!is_q && !write_cache) continue;
    const T* src = row + size_t(hh) * dim;     // the key heads follow the query heads
    const float* gain = is_q ? q_gain : k_gain;
    T* dst = is_q ? q_out + (size_t(t) * heads + hh) * dim
                  : k_pool + kv_offset(page, hh - heads, in_page, kv_heads, dim);
    float rstd = 1.f;
    if (gain) {
      float ss = 0.f;
      for (int e = lane; e < dim; e += 32) {
        const float v = to_f(src[e]);
        ss = fmaf(v, v, ss);
      }
      rstd = 1.0f / sqrtf(warp_sum(ss) / float(dim) + eps);
    }
    for (int e = lane; e < dim; e += 32) dst[e] = gain ? from_f<T>(to_f(src[e]) * rstd * gain[e]) : src[e];
  }
  if (write_cache) {
    const T* vsrc = row + size_t(heads + kv_heads) * dim;
    for (int i = threadIdx.x; i < kv_heads * v_dim; i += blockDim.x) {
      const int g = i / v_dim, e = i % v_dim;
      v_pool[kv_offset(page, g, in_page, kv_heads, v_dim) + e] = vsrc[i];
    }
  }
}

size_t raise_smem(const void* fn, size_t smem, size_t& configured) {
  if (smem > configured) {
    if (cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) return 0;
    configured = smem;
  }
  return smem;
}

constexpr size_t SMEM_MOST = 200 * 1024;

// value columns of a block of the scan and chunk-sum kernels: 64, or 32 where values are that short or
// a [dim][64] tile of S does not fit shared memory
int scan_columns(int dim, int v_dim) {
  int vb = v_dim > 32 ? 64 : 32;
  while (vb > 32 && (size_t(dim) * vb + 2 * size_t(dim)) * sizeof(float) > SMEM_MOST) vb /= 2;
  return vb;
}

}  // namespace

// act: 0 none, 1 silu on q, k and v. out: float32 [n_tokens, heads * v_dim].
PTB_API int ptb_linear_attention_scan(int dtype, const void* proj, int stride, float* state, int state_stride,
                                      const int* slots, const StepBatch* sb, const float* decay, float* out, int heads,
                                      int dim, int v_dim, int act, cudaStream_t stream) {
  if (sb->n_tokens <= 0) return PTB_OK;
  if (heads <= 0 || heads > 65535 || dim <= 0 || v_dim <= 0 || stride < 2 * heads * dim + heads * v_dim) return PTB_ERR_SIZE;
  const int vb = scan_columns(dim, v_dim);
  const size_t smem = (size_t(dim) * vb + 2 * size_t(dim)) * sizeof(float);
  if (smem > SMEM_MOST) return PTB_ERR_SIZE;
  dim3 grid(sb->n_seqs, heads, (v_dim + vb - 1) / vb);
  if (dtype == PTB_F32) {
    static size_t configured = 48 * 1024;
    if (!raise_smem((const void*)linear_attention_scan_kernel<float>, smem, configured)) return PTB_ERR_LAUNCH;
    linear_attention_scan_kernel<float><<<grid, vb, smem, stream>>>((const float*)proj, stride, state, state_stride, slots,
                                                                    *sb, decay, out, heads, dim, v_dim, act);
  } else if (dtype == PTB_BF16) {
    static size_t configured = 48 * 1024;
    if (!raise_smem((const void*)linear_attention_scan_kernel<__nv_bfloat16>, smem, configured)) return PTB_ERR_LAUNCH;
    linear_attention_scan_kernel<__nv_bfloat16><<<grid, vb, smem, stream>>>(
        (const __nv_bfloat16*)proj, stride, state, state_stride, slots, *sb, decay, out, heads, dim, v_dim, act);
  } else {
    return PTB_ERR_DTYPE;
  }
  return launch_status();
}

// The same for a step in which every sequence brings one token (the caller's word: `sb` is not read on the host).
PTB_API int ptb_linear_attention_token(int dtype, const void* proj, int stride, float* state, int state_stride,
                                       const int* slots, const StepBatch* sb, const float* decay, float* out, int heads,
                                       int dim, int v_dim, int act, cudaStream_t stream) {
  if (sb->n_tokens <= 0) return PTB_OK;
  if (sb->n_tokens != sb->n_seqs) return PTB_ERR_SIZE;
  if (heads <= 0 || heads > 65535 || dim <= 0 || v_dim <= 0 || stride < 2 * heads * dim + heads * v_dim || dim > 4096)
    return PTB_ERR_SIZE;
  const int threads = 512;
  int vj = 32;
  while (vj < 128 && vj < v_dim) vj *= 2;
  const size_t smem = (2 * size_t(dim) + threads) * sizeof(float);
  dim3 grid(sb->n_seqs, heads, (v_dim + vj - 1) / vj);
  if (dtype == PTB_F32)
    linear_attention_token_kernel<float><<<grid, threads, smem, stream>>>((const float*)proj, stride, state, state_stride,
                                                                          slots, *sb, decay, out, heads, dim, v_dim, act, vj);
  else if (dtype == PTB_BF16)
    linear_attention_token_kernel<__nv_bfloat16><<<grid, threads, smem, stream>>>(
        (const __nv_bfloat16*)proj, stride, state, state_stride, slots, *sb, decay, out, heads, dim, v_dim, act, vj);
  else
    return PTB_ERR_DTYPE;
  return launch_status();
}

PTB_API int ptb_linear_attention_chunk_tokens() { return CH; }

// Does the chunked form take these sizes (its third pass holds a chunk's queries, keys and scores in shared memory)?
PTB_API int ptb_linear_attention_chunks_supports(int dim, int v_dim) {
  const size_t smem = (2 * size_t(CH) * (dim + 1) + size_t(CH) * (CH + 1) + CH + 1) * sizeof(float);
  return (smem <= SMEM_MOST && (size_t(dim) * scan_columns(dim, v_dim) + 2 * size_t(dim)) * sizeof(float) <= SMEM_MOST) ? 1 : 0;
}

// sums: float32 scratch [n_chunks, heads, dim, v_dim]. The three passes in order on `stream`.
PTB_API int ptb_linear_attention_chunks(int dtype, const void* proj, int stride, float* state, int state_stride,
                                        const int* slots, const StepBatch* sb, const int* chunk_seq, const int* chunk_q0,
                                        const int* seq_chunk0, int n_chunks, const float* decay, float* sums, float* out,
                                        int heads, int dim, int v_dim, int act, cudaStream_t stream) {
  if (sb->n_tokens <= 0 || n_chunks <= 0) return PTB_OK;
  if (heads <= 0 || heads > 65535 || dim <= 0 || v_dim <= 0 || stride < 2 * heads * dim + heads * v_dim ||
      !ptb_linear_attention_chunks_supports(dim, v_dim) || sb->n_seqs > 65535)
    return PTB_ERR_SIZE;
  const int vb = scan_columns(dim, v_dim);
  const size_t smem1 = (size_t(dim) * vb + size_t(dim)) * sizeof(float);
  const size_t smem3 = (2 * size_t(CH) * (dim + 1) + size_t(CH) * (CH + 1) + CH + 1) * sizeof(float);
  dim3 grid1(n_chunks, heads, (v_dim + vb - 1) / vb), grid3(n_chunks, heads);
  const size_t per = size_t(heads) * dim * v_dim;
  dim3 grid2(unsigned((per + 255) / 256), sb->n_seqs);
#define PTB_LA_CHUNKS(TT)                                                                                              \
  {                                                                                                                    \
    static size_t c1 = 48 * 1024, c3 = 48 * 1024;                                                                      \
    if (!raise_smem((const void*)linear_attention_chunk_sum_kernel<TT>, smem1, c1)) return PTB_ERR_LAUNCH;             \
    if (!raise_smem((const void*)linear_attention_chunk_out_kernel<TT>, smem3, c3)) return PTB_ERR_LAUNCH;             \
    linear_attention_chunk_sum_kernel<TT><<<grid1, vb, smem1, stream>>>((const TT*)proj, stride, *sb, chunk_seq,        \
                                                                        chunk_q0, decay, sums, heads, dim, v_dim, act); \
    if (launch_status() != PTB_OK) return PTB_ERR_LAUNCH;                                                              \
    linear_attention_chunk_join_kernel<<<grid2, 256, 0, stream>>>(sums, state, state_stride, slots, *sb, seq_chunk0,   \
                                                                  decay, heads, dim, v_dim);                           \
    if (launch_status() != PTB_OK) return PTB_ERR_LAUNCH;                                                              \
    linear_attention_chunk_out_kernel<TT><<<grid3, 256, smem3, stream>>>((const TT*)proj, stride, *sb, chunk_seq,       \
                                                                         chunk_q0, decay, sums, out, heads, dim, v_dim, \
                                                                         act);                                         \
  }
  if (dtype == PTB_F32) PTB_LA_CHUNKS(float)
  else if (dtype == PTB_BF16) PTB_LA_CHUNKS(__nv_bfloat16)
  else return PTB_ERR_DTYPE;
#undef PTB_LA_CHUNKS
  return launch_status();
}

// pass 2 alone (the tensor-core passes 1 and 3 are in csrc/linear_attention_mma.cu)
PTB_API int ptb_linear_attention_chunk_join(float* sums, float* state, int state_stride, const int* slots,
                                            const StepBatch* sb, const int* seq_chunk0, const float* decay, int heads,
                                            int dim, int v_dim, cudaStream_t stream) {
  if (sb->n_tokens <= 0) return PTB_OK;
  if (heads <= 0 || dim <= 0 || v_dim <= 0 || sb->n_seqs > 65535) return PTB_ERR_SIZE;
  const size_t per = size_t(heads) * dim * v_dim;
  dim3 grid(unsigned((per + 255) / 256), sb->n_seqs);
  linear_attention_chunk_join_kernel<<<grid, 256, 0, stream>>>(sums, state, state_stride, slots, *sb, seq_chunk0, decay,
                                                               heads, dim, v_dim);
  return launch_status();
}

PTB_API int ptb_norm_gate(const float* x, const float* gain, int gate_dtype, const void* gate, int gate_stride,
                          int out_dtype, void* y, int y_stride, int n, int width, float eps, float out_scale,
                          cudaStream_t stream) {
  if (n <= 0) return PTB_OK;
  if (width <= 0 || y_stride < width || (gate != nullptr && gate_stride < width)) return PTB_ERR_SIZE;
  if (gate_dtype != out_dtype) return PTB_ERR_DTYPE;
  const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
  if (out_dtype == PTB_F32)
    norm_gate_kernel<float, float><<<n, threads, 0, stream>>>(x, gain, (const float*)gate, gate_stride, (float*)y,
                                                              y_stride, width, eps, out_scale);
  else if (out_dtype == PTB_BF16)
    norm_gate_kernel<__nv_bfloat16, __nv_bfloat16><<<n, threads, 0, stream>>>(
        x, gain, (const __nv_bfloat16*)gate, gate_stride, (__nv_bfloat16*)y, y_stride, width, eps, out_scale);
  else
    return PTB_ERR_DTYPE;
  return launch_status();
}

// q_gain / k_gain: float32 [dim] or null (no norm of queries and keys)
PTB_API int ptb_qk_norm_store(int dtype, const void* proj, int stride, void* q_out, void* k_pool, void* v_pool,
                              const StepBatch* sb, const float* q_gain, const float* k_gain, int heads, int kv_heads,
                              int dim, int v_dim, float eps, int write_cache, cudaStream_t stream) {
  if (sb->n_tokens <= 0) return PTB_OK;
  if (heads <= 0 || kv_heads <= 0 || dim <= 0 || v_dim <= 0 || stride < (heads + kv_heads) * dim + kv_heads * v_dim ||
      (q_gain == nullptr) != (k_gain == nullptr))
    return PTB_ERR_SIZE;
  const int threads = 256;
  if (dtype == PTB_F32)
    qk_norm_store_kernel<float><<<sb->n_tokens, threads, 0, stream>>>((const float*)proj, stride, (float*)q_out,
                                                                      (float*)k_pool, (float*)v_pool, *sb, q_gain, k_gain,
                                                                      heads, kv_heads, dim, v_dim, eps, write_cache);
  else if (dtype == PTB_BF16)
    qk_norm_store_kernel<__nv_bfloat16><<<sb->n_tokens, threads, 0, stream>>>(
        (const __nv_bfloat16*)proj, stride, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, *sb,
        q_gain, k_gain, heads, kv_heads, dim, v_dim, eps, write_cache);
  else
    return PTB_ERR_DTYPE;
  return launch_status();
}
