// The gated linear recurrence block (two branches, a short causal convolution, block-diagonal
// gates, a diagonal recurrence with per-sequence state) and the block-diagonal linear layer that
// its gates and the latent attention's per-head projections use.
//
// Per-sequence state of a layer, float32, one row per cache slot:
//   [0, R)                      the recurrence's state S
//   [R + k R, R + (k + 1) R)    the convolution's input at position length - (taps - 1) + k, k < taps - 1
// (zero for a sequence that has just started, which is the convolution's zero padding and S = 0).
#include "common.cuh"

namespace {

constexpr int MAX_TAPS = 8;

// proj [tokens, 2 R]: columns [0, R) the gate branch before its bias, [R, 2 R) the recurrent branch
// before its bias. Writes y_act = gelu_tanh(gate branch + by) and u = conv(recurrent branch + bx):
//   u[t, c] = conv_b[c] + sum_k conv_w[c, k] * in[t - (taps - 1) + k, c]
// with inputs before the step's first token taken from the state. One thread per (token, channel).
template <typename T>
__global__ void rglru_conv_kernel(const T* __restrict__ proj, const float* __restrict__ by,
                                  const float* __restrict__ bx, const float* __restrict__ conv_w,
                                  const float* __restrict__ conv_b, const float* __restrict__ state,
                                  long long state_stride, const int* __restrict__ slots, StepBatch sb,
                                  T* __restrict__ y_act, T* __restrict__ u, int R, int taps) {
  const size_t total = size_t(sb.n_tokens) * R, stride = size_t(gridDim.x) * blockDim.x;
  for (size_t idx = size_t(blockIdx.x) * blockDim.x + threadIdx.x; idx < total; idx += stride) {
    const int t = int(idx / R), c = int(idx % R);
    const int seq = sb.tok_seq[t];
    const int local = t - sb.seq_start[seq];
    const float* hist = state + size_t(slots[seq]) * state_stride + R;
    float acc = conv_b[c];
    for (int k = 0; k < taps; ++k) {
      const int j = local - (taps - 1) + k;
      const float v = (j >= 0) ? to_f(proj[size_t(t - local + j) * 2 * R + R + c]) + bx[c]
                               : hist[size_t(j + taps - 1) * R + c];
      acc = fmaf(conv_w[size_t(c) * taps + k], v, acc);
    }
    u[idx] = from_f<T>(acc);
    y_act[idx] = from_f<T>(apply_activation(to_f(proj[size_t(t) * 2 * R + c]) + by[c], PTB_ACT_GELU_TANH));
  }
}

// a S + drive with a = exp(log_a), formed as S + ((a - 1) S + drive) with a - 1 = expm1(log_a): a decay close
// to 1 rounded to float32 is off by up to 3e-8 of itself, which a channel whose decay hardly changes would
// carry into every step alike (1,000 steps: 3e-5 of the state); a - 1 keeps its digits, and what is left is
// the rounding of the sum, which does not add up in one direction.
__device__ __forceinline__ float decayed(float S, float log_a, float drive) {
  return S + fmaf(expm1f(log_a), S, drive);
}

// One thread per (sequence, channel) walks the sequence's new tokens in order:
//   log a = -c_decay * r * softplus(lam),  a = exp(log a)
//   S <- a S + sqrt(1 - a^2) * (i * u),    out = S * y_act
// gates [tokens, blocks, 2 * bw] float32 hold r (first bw of a block) and i (last bw) after their
// sigmoid. All of it in float32; 1 - a^2 is formed as -expm1(2 log a). At the end the state takes S
// and the last taps - 1 inputs of the convolution.
template <typename T>
__global__ void rglru_scan_kernel(const float* __restrict__ gates, const T* __restrict__ u,
                                  const T* __restrict__ y_act, const float* __restrict__ lam,
                                  const T* __restrict__ proj, const float* __restrict__ bx, float* __restrict__ state,
                                  long long state_stride, const int* __restrict__ slots, StepBatch sb,
                                  T* __restrict__ out, int R, int bw, int taps, float c_decay) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= sb.n_seqs * R) return;
  const int seq = idx / R, c = idx % R;
  const int start = sb.seq_start[seq], n_new = sb.seq_new[seq];
  float* st = state + size_t(slots[seq]) * state_stride;
  const float l = lam[c];
  const float sp = (l > 20.f) ? l : log1pf(expf(l));
  const int g = c / bw, j = c % bw;
  const size_t goff = size_t(g) * 2 * bw + j;
  float S = st[c];
  for (int i = 0; i < n_new; ++i) {
    const size_t t = size_t(start + i);
    const float r = gates[t * 2 * R + goff], in = gates[t * 2 * R + goff + bw];
    const float log_a = -c_decay * r * sp;
    const float drive = sqrtf(-expm1f(2.f * log_a)) * (in * to_f(u[t * R + c]));
    S = decayed(S, log_a, drive);
    out[t * R + c] = from_f<T>(S * to_f(y_act[t * R + c]));
  }
  st[c] = S;
  float keep[MAX_TAPS];
  for (int k = 0; k < taps - 1; ++k) {
    const int jj = n_new - (taps - 1) + k;
    keep[k] = (jj >= 0) ? to_f(proj[size_t(start + jj) * 2 * R + R + c]) + bx[c] : st[R + size_t(jj + taps - 1) * R + c];
  }
  for (int k = 0; k < taps - 1; ++k) st[R + size_t(k) * R + c] = keep[k];
}

// The same recurrence for long prompts, cut into chunks of consecutive tokens of one sequence so that the
// chunks run side by side: S_end = A S_start + B with A the product of a chunk's decays (kept as the sum of
// their logarithms) and B its result
// from S_start = 0. Pass 1 (a thread per chunk and channel) finds (A, B) of every chunk; pass 2 (a thread
// per sequence and channel) walks a sequence's chunks in order, notes every chunk's S_start, and leaves
// the state (S and the convolution's last inputs); pass 3 (a thread per chunk and channel) runs the
// chunk again from its S_start and writes the outputs. PASS selects the pass.
template <typename T, int PASS>
__global__ void rglru_chunk_kernel(const float* __restrict__ gates, const T* __restrict__ u, const T* __restrict__ y_act,
                                   const float* __restrict__ lam, const T* __restrict__ proj,
                                   const float* __restrict__ bx, float* __restrict__ state, long long state_stride,
                                   const int* __restrict__ slots, StepBatch sb, const int* __restrict__ chunk_seq,
                                   const int* __restrict__ chunk_q0, const int* __restrict__ seq_chunk0, int n_chunks,
                                   int chunk_len, float* __restrict__ agg_a, float* __restrict__ agg_b,
                                   float* __restrict__ s_start, T* __restrict__ out, int R, int bw, int taps,
                                   float c_decay) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= R) return;
  if (PASS == 2) {
    const int seq = blockIdx.y;
    const int n_new = sb.seq_new[seq], start = sb.seq_start[seq];
    float* st = state + size_t(slots[seq]) * state_stride;
    float S = st[c];
    const int first = seq_chunk0[seq], count = (n_new + chunk_len - 1) / chunk_len;
    for (int k = first; k < first + count; ++k) {
      s_start[size_t(k) * R + c] = S;
      S = decayed(S, agg_a[size_t(k) * R + c], agg_b[size_t(k) * R + c]);     // agg_a holds the chunk's summed log a
    }
    st[c] = S;
    float keep[MAX_TAPS];
    for (int k = 0; k < taps - 1; ++k) {
      const int jj = n_new - (taps - 1) + k;
      keep[k] = (jj >= 0) ? to_f(proj[size_t(start + jj) * 2 * R + R + c]) + bx[c] : st[R + size_t(jj + taps - 1) * R + c];
    }
    for (int k = 0; k < taps - 1; ++k) st[R + size_t(k) * R + c] = keep[k];
    return;
  }
  const int chunk = blockIdx.y;
  const int seq = chunk_seq[chunk], q0 = chunk_q0[chunk];
  const int first = sb.seq_start[seq] + q0, count = min(chunk_len, sb.seq_new[seq] - q0);
  const float l = lam[c];
  const float sp = (l > 20.f) ? l : log1pf(expf(l));
  const size_t goff = size_t(c / bw) * 2 * bw + c % bw;
  float S = (PASS == 3) ? s_start[size_t(chunk) * R + c] : 0.f, A = 0.f;      // A: the chunk's summed log a
  for (int i = 0; i < count; ++i) {
    const size_t t = size_t(first + i);
    const float r = gates[t * 2 * R + goff], in = gates[t * 2 * R + goff + bw];
    const float log_a = -c_decay * r * sp;
    S = decayed(S, log_a, sqrtf(-expm1f(2.f * log_a)) * (in * to_f(u[t * R + c])));
    if (PASS == 1) A += log_a;
    if (PASS == 3) out[t * R + c] = from_f<T>(S * to_f(y_act[t * R + c]));
  }
  if (PASS == 1) {
    agg_a[size_t(chunk) * R + c] = A;
    agg_b[size_t(chunk) * R + c] = S;
  }
}

template <typename T>
int launch_rglru_chunks(const float* gates, const void* u, const void* y_act, const float* lam, const void* proj,
                        const float* bx, float* state, long long state_stride, const int* slots, const StepBatch& sb,
                        const int* chunk_seq, const int* chunk_q0, const int* seq_chunk0, int n_chunks, int chunk_len,
                        float* work, void* out, int R, int bw, int taps, float c_decay, cudaStream_t stream) {
  float* agg_a = work;
  float* agg_b = work + size_t(n_chunks) * R;
  float* s_start = work + 2 * size_t(n_chunks) * R;
  const int threads = 128, gx = (R + threads - 1) / threads;
#define PTB_CHUNK_PASS(P, GY)                                                                                      \
  rglru_chunk_kernel<T, P><<<dim3(gx, GY), threads, 0, stream>>>(                                                   \
      gates, (const T*)u, (const T*)y_act, lam, (const T*)proj, bx, state, state_stride, slots, sb, chunk_seq, chunk_q0, \
      seq_chunk0, n_chunks, chunk_len, agg_a, agg_b, s_start, (T*)out, R, bw, taps, c_decay)
  PTB_CHUNK_PASS(1, n_chunks);
  PTB_CHUNK_PASS(2, sb.n_seqs);
  PTB_CHUNK_PASS(3, n_chunks);
#undef PTB_CHUNK_PASS
  return launch_status();
}

// y[t, g, :] = act(W[g] x[t, g, :] + bias[g]) [* sigmoid(gate[t, g, :])], W [groups, N, K]; x is read with
// strides (a token's stride xt, a group's stride xg), y [tokens, groups, N] is float32 or the input's
// type. float32 FMAs in ascending k, 16 products summed apart and then into the total: a row's
// result does not depend on the other rows of the launch. act: 0 none, 1 sigmoid.
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename T, typename TO>
__global__ void __launch_bounds__(256)
block_linear_kernel(const T* __restrict__ x, long long xt, long long xg, const T* __restrict__ w,
                    const float* __restrict__ bias, TO* __restrict__ y, const T* __restrict__ gate, long long gate_t,
                    int M, int G, int N, int K, int act) {
  __shared__ float xs[BK][BM + 4];
  __shared__ float ws[BK][BN + 4];
  const int tid = threadIdx.x, g = blockIdx.z;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tm = (tid / 16) * TM, tn = (tid % 16) * TN;
  const int lrow = tid / 4, lk = (tid % 4) * 4;
  const T* wg = w + size_t(g) * N * K;
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int k = k0 + lk + q;
      const int gm = m0 + lrow, gn = n0 + lrow;
      xs[lk + q][lrow] = (gm < M && k < K) ? to_f(x[size_t(gm) * xt + size_t(g) * xg + k]) : 0.f;
      ws[lk + q][lrow] = (gn < N && k < K) ? to_f(wg[size_t(gn) * K + k]) : 0.f;
    }
    __syncthreads();
    float part[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
      for (int j = 0; j < TN; ++j) part[i][j] = 0.f;
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = xs[k][tm + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = ws[k][tn + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) part[i][j] = fmaf(a[i], b[j], part[i][j]);
    }
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
      for (int j = 0; j < TN; ++j) acc[i][j] += part[i][j];
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int gm = m0 + tm + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int gn = n0 + tn + j;
      if (gn >= N) continue;
      float v = acc[i][j];
      if (bias) v += bias[size_t(g) * N + gn];
      if (act == 1) v = 1.f / (1.f + expf(-v));
      if (gate) v *= 1.f / (1.f + expf(-to_f(gate[size_t(gm) * gate_t + size_t(g) * N + gn])));
      y[(size_t(gm) * G + g) * N + gn] = from_f<TO>(v);
    }
  }
}

// The same for a few rows (steps of single tokens): a warp per (group, output) reads its row of W once,
// lanes along K, and forms the sums of all M <= 16 rows; the order of a row's sums is fixed.
constexpr int SKINNY_M = 16;
template <typename T> __device__ __forceinline__ void load8(const T* p, float (&f)[8], bool vec);
template <> __device__ __forceinline__ void load8<float>(const float* p, float (&f)[8], bool) {
#pragma unroll
  for (int i = 0; i < 8; ++i) f[i] = p[i];
}
template <> __device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&f)[8], bool vec) {
  if (vec) {
    unpack_bf16x8(*reinterpret_cast<const uint4*>(p), f);
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = __bfloat162float(p[i]);
  }
}

// `vec`: every row of x and w starts on a 16-byte boundary and K is a multiple of 8 (the host checks):
// bfloat16 operands then move in 16-byte words. A lane takes 8 consecutive k at a time.
template <typename T, typename TO>
__global__ void __launch_bounds__(256)
block_linear_skinny_kernel(const T* __restrict__ x, long long xt, long long xg, const T* __restrict__ w,
                           const float* __restrict__ bias, TO* __restrict__ y, const T* __restrict__ gate,
                           long long gate_t, int M, int G, int N, int K, int act, int vec) {
  const int lane = threadIdx.x % 32;
  const long long item = (long long)blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
  if (item >= (long long)G * N) return;
  const int g = int(item / N), n = int(item % N);
  const T* wr = w + (size_t(g) * N + n) * K;
  float acc[SKINNY_M];
#pragma unroll
  for (int m = 0; m < SKINNY_M; ++m) acc[m] = 0.f;
  const int k_whole = K / 8 * 8;
  for (int k = lane * 8; k < k_whole; k += 256) {
    float wv[8];
    load8<T>(wr + k, wv, vec);
#pragma unroll
    for (int m = 0; m < SKINNY_M; ++m) {
      if (m < M) {
        float xv[8];
        load8<T>(x + size_t(m) * xt + size_t(g) * xg + k, xv, vec);
        float part = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) part = fmaf(wv[i], xv[i], part);
        acc[m] += part;
      }
    }
  }
  for (int k = k_whole + lane; k < K; k += 32) {
    const float wv = to_f(wr[k]);
#pragma unroll
    for (int m = 0; m < SKINNY_M; ++m)
      if (m < M) acc[m] = fmaf(wv, to_f(x[size_t(m) * xt + size_t(g) * xg + k]), acc[m]);
  }
#pragma unroll
  for (int m = 0; m < SKINNY_M; ++m) {
    if (m >= M) break;
    float v = warp_sum(acc[m]);
    if (lane == 0) {
      if (bias) v += bias[size_t(g) * N + n];
      if (act == 1) v = 1.f / (1.f + expf(-v));
      if (gate) v *= 1.f / (1.f + expf(-to_f(gate[size_t(m) * gate_t + size_t(g) * N + n])));
      y[(size_t(m) * G + g) * N + n] = from_f<TO>(v);
    }
  }
}

// The epilogue of block_linear for products that the library's batched routine made: z [groups, M, N]
// (float32 or bfloat16) -> y [M, groups, N] = act(z + bias[g]) [* sigmoid(gate)], float32 sums.
template <typename TI, typename TO, typename TG>
__global__ void block_epilogue_kernel(const TI* __restrict__ z, const float* __restrict__ bias, const TG* __restrict__ gate,
                                      long long gate_t, TO* __restrict__ y, int M, int G, int N, int act) {
  const size_t total = size_t(M) * G * N, stride = size_t(gridDim.x) * blockDim.x;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int n = int(i % N), g = int((i / N) % G), m = int(i / (size_t(N) * G));
    float v = to_f(z[(size_t(g) * M + m) * N + n]);
    if (bias) v += bias[size_t(g) * N + n];
    if (act == 1) v = 1.f / (1.f + expf(-v));
    if (gate) v *= 1.f / (1.f + expf(-to_f(gate[size_t(m) * gate_t + size_t(g) * N + n])));
    y[i] = from_f<TO>(v);
  }
}

}  // namespace

PTB_API int ptb_block_epilogue(int in_dtype, int out_dtype, const void* z, const float* bias, const void* gate,
                               long long gate_t, void* y, int M, int G, int N, int act, cudaStream_t stream) {
  if (M <= 0 || G <= 0 || N <= 0) return PTB_OK;
  if (act < 0 || act > 1) return PTB_ERR_SIZE;
  const size_t total = size_t(M) * G * N, want = (total + 255) / 256, most = size_t(sm_count()) * 16;
  const int blocks = int(want < most ? want : most);
  typedef __nv_bfloat16 bf;
  if (in_dtype == PTB_F32 && out_dtype == PTB_F32)
    block_epilogue_kernel<float, float, bf><<<blocks, 256, 0, stream>>>((const float*)z, bias, (const bf*)gate, gate_t, (float*)y, M, G, N, act);
  else if (in_dtype == PTB_F32 && out_dtype == PTB_BF16)
    block_epilogue_kernel<float, bf, bf><<<blocks, 256, 0, stream>>>((const float*)z, bias, (const bf*)gate, gate_t, (bf*)y, M, G, N, act);
  else if (in_dtype == PTB_BF16 && out_dtype == PTB_BF16)
    block_epilogue_kernel<bf, bf, bf><<<blocks, 256, 0, stream>>>((const bf*)z, bias, (const bf*)gate, gate_t, (bf*)y, M, G, N, act);
  else if (in_dtype == PTB_BF16 && out_dtype == PTB_F32)
    block_epilogue_kernel<bf, float, bf><<<blocks, 256, 0, stream>>>((const bf*)z, bias, (const bf*)gate, gate_t, (float*)y, M, G, N, act);
  else
    return PTB_ERR_DTYPE;
  return launch_status();
}

PTB_API int ptb_rglru_conv(int dtype, const void* proj, const float* by, const float* bx, const float* conv_w,
                           const float* conv_b, const float* state, long long state_stride, const int* slots,
                           const StepBatch* sb, void* y_act, void* u, int R, int taps, cudaStream_t stream) {
  if (sb->n_tokens <= 0) return PTB_OK;
  if (R <= 0 || taps < 1 || taps > MAX_TAPS) return PTB_ERR_SIZE;
  const size_t total = size_t(sb->n_tokens) * R;
  const size_t want = (total + 255) / 256, most = size_t(sm_count()) * 16;
  const int blocks = int(want < most ? want : most);
  if (dtype == PTB_F32)
    rglru_conv_kernel<float><<<blocks, 256, 0, stream>>>((const float*)proj, by, bx, conv_w, conv_b, state,
                                                         state_stride, slots, *sb, (float*)y_act, (float*)u, R, taps);
  else if (dtype == PTB_BF16)
    rglru_conv_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)proj, by, bx, conv_w, conv_b,
                                                                 state, state_stride, slots, *sb,
                                                                 (__nv_bfloat16*)y_act, (__nv_bfloat16*)u, R, taps);
  else
    return PTB_ERR_DTYPE;
  return launch_status();
}

PTB_API int ptb_rglru_scan(int dtype, const float* gates, const void* u, const void* y_act, const float* lam,
                           const void* proj, const float* bx, float* state, long long state_stride, const int* slots,
                           const StepBatch* sb, void* out, int R, int blocks_n, int taps, float c_decay,
                           cudaStream_t stream) {
  if (sb->n_tokens <= 0) return PTB_OK;
  if (R <= 0 || blocks_n <= 0 || R % blocks_n != 0 || taps < 1 || taps > MAX_TAPS) return PTB_ERR_SIZE;
  const int bw = R / blocks_n;
  const int total = sb->n_seqs * R;
  const int threads = 128, grid = (total + threads - 1) / threads;
  if (dtype == PTB_F32)
    rglru_scan_kernel<float><<<grid, threads, 0, stream>>>(gates, (const float*)u, (const float*)y_act, lam,
                                                           (const float*)proj, bx, state, state_stride, slots, *sb,
                                                           (float*)out, R, bw, taps, c_decay);
  else if (dtype == PTB_BF16)
    rglru_scan_kernel<__nv_bfloat16><<<grid, threads, 0, stream>>>(
        gates, (const __nv_bfloat16*)u, (const __nv_bfloat16*)y_act, lam, (const __nv_bfloat16*)proj, bx, state,
        state_stride, slots, *sb, (__nv_bfloat16*)out, R, bw, taps, c_decay);
  else
    return PTB_ERR_DTYPE;
  return launch_status();
}

// `work`: 3 * n_chunks * R float32 values
PTB_API int ptb_rglru_scan_chunks(int dtype, const float* gates, const void* u, const void* y_act, const float* lam,
                                  const void* proj, const float* bx, float* state, long long state_stride,
                                  const int* slots, const StepBatch* sb, const int* chunk_seq, const int* chunk_q0,
                                  const int* seq_chunk0, int n_chunks, int chunk_len, float* work, void* out, int R,
                                  int blocks_n, int taps, float c_decay, cudaStream_t stream) {
  if (sb->n_tokens <= 0 || n_chunks <= 0) return PTB_OK;
  if (R <= 0 || blocks_n <= 0 || R % blocks_n != 0 || taps < 1 || taps > MAX_TAPS || chunk_len <= 0 ||
      n_chunks > 65535 || sb->n_seqs > 65535)
    return PTB_ERR_SIZE;
  if (dtype == PTB_F32)
    return launch_rglru_chunks<float>(gates, u, y_act, lam, proj, bx, state, state_stride, slots, *sb, chunk_seq,
                                      chunk_q0, seq_chunk0, n_chunks, chunk_len, work, out, R, R / blocks_n, taps,
                                      c_decay, stream);
  if (dtype == PTB_BF16)
    return launch_rglru_chunks<__nv_bfloat16>(gates, u, y_act, lam, proj, bx, state, state_stride, slots, *sb,
                                              chunk_seq, chunk_q0, seq_chunk0, n_chunks, chunk_len, work, out, R,
                                              R / blocks_n, taps, c_decay, stream);
  return PTB_ERR_DTYPE;
}

PTB_API int ptb_block_linear(int dtype, int out_dtype, const void* x, long long xt, long long xg, const void* w,
                             const float* bias, void* y, const void* gate, long long gate_t, int M, int G, int N,
                             int K, int act, cudaStream_t stream) {
  if (M <= 0 || G <= 0 || N <= 0) return PTB_OK;
  if (K <= 0 || act < 0 || act > 1 || G > 65535) return PTB_ERR_SIZE;
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM, G);
  if (grid.y > 65535) return PTB_ERR_SIZE;
  if (M <= SKINNY_M) {
    const long long items = (long long)G * N;
    const int sgrid = int((items + 7) / 8);
    typedef __nv_bfloat16 bf;
    const int vec = (K % 8 == 0 && xt % 8 == 0 && xg % 8 == 0 && aligned16(x) && aligned16(w)) ? 1 : 0;
    if (dtype == PTB_F32 && out_dtype == PTB_F32)
      block_linear_skinny_kernel<float, float><<<sgrid, 256, 0, stream>>>((const float*)x, xt, xg, (const float*)w, bias, (float*)y, (const float*)gate, gate_t, M, G, N, K, act, vec);
    else if (dtype == PTB_BF16 && out_dtype == PTB_F32)
      block_linear_skinny_kernel<bf, float><<<sgrid, 256, 0, stream>>>((const bf*)x, xt, xg, (const bf*)w, bias, (float*)y, (const bf*)gate, gate_t, M, G, N, K, act, vec);
    else if (dtype == PTB_BF16 && out_dtype == PTB_BF16)
      block_linear_skinny_kernel<bf, bf><<<sgrid, 256, 0, stream>>>((const bf*)x, xt, xg, (const bf*)w, bias, (bf*)y, (const bf*)gate, gate_t, M, G, N, K, act, vec);
    else
      return PTB_ERR_DTYPE;
    return launch_status();
  }
  if (dtype == PTB_F32 && out_dtype == PTB_F32)
    block_linear_kernel<float, float><<<grid, 256, 0, stream>>>((const float*)x, xt, xg, (const float*)w, bias,
                                                                (float*)y, (const float*)gate, gate_t, M, G, N, K, act);
  else if (dtype == PTB_BF16 && out_dtype == PTB_F32)
    block_linear_kernel<__nv_bfloat16, float><<<grid, 256, 0, stream>>>(
        (const __nv_bfloat16*)x, xt, xg, (const __nv_bfloat16*)w, bias, (float*)y, (const __nv_bfloat16*)gate, gate_t,
        M, G, N, K, act);
  else if (dtype == PTB_BF16 && out_dtype == PTB_BF16)
    block_linear_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, 256, 0, stream>>>(
        (const __nv_bfloat16*)x, xt, xg, (const __nv_bfloat16*)w, bias, (__nv_bfloat16*)y, (const __nv_bfloat16*)gate,
        gate_t, M, G, N, K, act);
  else
    return PTB_ERR_DTYPE;
  return launch_status();
}
