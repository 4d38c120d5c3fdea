// Latent attention over the paged cache: every token caches one row [latent c (rank) | shared rotated
// key part (rot_dim)] that all heads read. With the key up-projection folded into the query
// (q_abs[h] = W_uk[h]^T q_plain[h]) a head's score against a cached row is
//   (q_abs[h] . c + q_rot[h] . k_rot) * scale
// and its output in latent space is sum_j p_j c_j; the value up-projection follows outside.
// So the heads of a token are rows of one tile over the same cached rows, and the values are the
// first `rank` entries of the keys: a page is staged once and used for scores and for outputs.
// All arithmetic is float32 on the CUDA cores; keys are reduced in blocks of 64 aligned to absolute
// positions in ascending order, so a position's result does not depend on how its tokens were cut
// into steps or batched.
#include "common.cuh"

namespace {

constexpr int ROWS = 16;      // (token, head) rows of a tile
constexpr int THREADS = 128;  // 8 threads per row

// One block per token: the row `src` [rank + rot_dim] of the down-projection becomes the cached row:
// the first `rank` entries divided by their root mean square (eps inside the root) times norm_w,
// the last rot_dim rotated by the token's position (pairs (2i, 2i+1) when interleaved, else
// (i, i + rot_pairs)); entries past 2 * rot_pairs pass unchanged.
template <typename T>
__global__ void latent_store_kernel(const T* __restrict__ src, long long src_stride, const float* __restrict__ norm_w,
                                    float eps, T* __restrict__ pool, StepBatch sb, const float* __restrict__ rope_cos,
                                    const float* __restrict__ rope_sin, int rot_pairs, int interleaved, int rank,
                                    int rot_dim) {
  __shared__ float scratch[32];
  const int t = blockIdx.x;
  const int pos = sb.tok_pos[t], seq = sb.tok_seq[t];
  const int page = sb.pages[size_t(seq) * sb.pages_stride + pos / PTB_PAGE];
  const T* row = src + size_t(t) * src_stride;
  T* dst = pool + kv_offset(page, 0, pos % PTB_PAGE, 1, rank + rot_dim);
  float q = 0.f;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) {
    const float v = to_f(row[i]);
    q += v * v;
  }
  const float rstd = 1.0f / sqrtf(block_sum(q, scratch) / float(rank) + eps);
  for (int i = threadIdx.x; i < rank; i += blockDim.x) dst[i] = from_f<T>(to_f(row[i]) * rstd * norm_w[i]);
  const int items = rot_pairs + (rot_dim - 2 * rot_pairs);
  for (int e = threadIdx.x; e < items; e += blockDim.x) {
    if (e < rot_pairs) {
      const int ia = interleaved ? 2 * e : e, ib = interleaved ? 2 * e + 1 : e + rot_pairs;
      float a, b;
      rotate_pair(to_f(row[rank + ia]), to_f(row[rank + ib]), rope_cos[size_t(t) * rot_pairs + e],
                  rope_sin[size_t(t) * rot_pairs + e], a, b);
      dst[rank + ia] = from_f<T>(a);
      dst[rank + ib] = from_f<T>(b);
    } else {
      const int i = 2 * rot_pairs + (e - rot_pairs);
      dst[rank + i] = row[rank + i];
    }
  }
}

// One block = one tile (tile_tokens consecutive new tokens of a sequence) x one chunk of
// heads_per_block heads x one split of the key pages; tile_tokens * heads_per_block <= ROWS.
//   q_abs [tokens, heads, rank] float32: queries with the key up-projection folded in
//   q     [tokens, heads, q_dim]: the projection's rows; the part to rotate starts at q_rot_off
//   pool  [pages][64][rank + rot_dim]
//   out   [tokens, heads, rank]: softmax-weighted sums of the latents
// With n_splits > 1 a block writes (max, sum, unnormalised sums) of its pages to `part` and
// latent_join_kernel merges the splits in order.
template <typename T, int DPT>
__global__ void __launch_bounds__(THREADS)
latent_attention_kernel(const float* __restrict__ q_abs, const T* __restrict__ q, int q_dim, int q_rot_off,
                        const T* __restrict__ pool, float* __restrict__ part, T* __restrict__ out, StepBatch sb,
                        const int* __restrict__ tile_seq, const int* __restrict__ tile_q0,
                        const float* __restrict__ rope_cos, const float* __restrict__ rope_sin, int rot_pairs,
                        int interleaved, int heads, int rank, int rot_dim, int tile_tokens, int heads_per_block,
                        float scale, int n_splits) {
  extern __shared__ float smem[];
  const int dk = rank + rot_dim, qstride = dk + 1, kstride = dk + 1;
  float* qs = smem;                       // [ROWS][dk + 1]
  float* kv = qs + ROWS * qstride;        // [64][dk + 1]
  float* ps = kv + PTB_PAGE * kstride;    // [ROWS][64]

  const int tile = blockIdx.x, h0 = blockIdx.y * heads_per_block, split = blockIdx.z;
  const int seq = tile_seq[tile], q0 = tile_q0[tile];
  const int n_new = sb.seq_new[seq], past = sb.seq_past[seq], start = sb.seq_start[seq];
  const int toks = min(tile_tokens, n_new - q0);
  const int tid = threadIdx.x, r = tid / 8, c = tid % 8;
  const int my_tok = r / heads_per_block, my_head = h0 + r % heads_per_block;
  const bool my_row = my_tok < toks && my_head < heads && r < tile_tokens * heads_per_block;
  const int my_pos = my_row ? past + q0 + my_tok : -1;

  for (int i = tid; i < ROWS * rank; i += THREADS) {
    const int rr = i / rank, e = i % rank;
    const int ti = rr / heads_per_block, hh = h0 + rr % heads_per_block;
    const bool ok = ti < toks && hh < heads && rr < tile_tokens * heads_per_block;
    qs[rr * qstride + e] = ok ? q_abs[(size_t(start + q0 + ti) * heads + hh) * rank + e] : 0.f;
  }
  const int items = rot_pairs + (rot_dim - 2 * rot_pairs);
  for (int i = tid; i < ROWS * items; i += THREADS) {
    const int rr = i / items, e = i % items;
    const int ti = rr / heads_per_block, hh = h0 + rr % heads_per_block;
    const bool ok = ti < toks && hh < heads && rr < tile_tokens * heads_per_block;
    const size_t tok = size_t(start + q0 + ti);
    const T* src = q + (tok * heads + hh) * q_dim + q_rot_off;
    float* dst = qs + rr * qstride + rank;
    if (e < rot_pairs) {
      const int ia = interleaved ? 2 * e : e, ib = interleaved ? 2 * e + 1 : e + rot_pairs;
      float a = 0.f, b = 0.f;
      if (ok) rotate_pair(to_f(src[ia]), to_f(src[ib]), rope_cos[tok * rot_pairs + e], rope_sin[tok * rot_pairs + e], a, b);
      dst[ia] = a;
      dst[ib] = b;
    } else {
      const int j = 2 * rot_pairs + (e - rot_pairs);
      dst[j] = ok ? to_f(src[j]) : 0.f;
    }
  }

  float acc[DPT];
#pragma unroll
  for (int i = 0; i < DPT; ++i) acc[i] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;

  const int last_pos = past + q0 + toks - 1;
  const int n_blocks = last_pos / PTB_PAGE + 1;
  const int per = (n_blocks + n_splits - 1) / n_splits;
  const int kb_lo = split * per, kb_hi = min(n_blocks, kb_lo + per) - 1;
  const int* pages = sb.pages + size_t(seq) * sb.pages_stride;
  const bool vec = sizeof(T) == 2 && dk % 8 == 0 && aligned16(pool);

  for (int kb = kb_lo; kb <= kb_hi; ++kb) {
    const int valid = min(PTB_PAGE, last_pos + 1 - kb * PTB_PAGE);
    const T* kp = pool + kv_offset(pages[kb], 0, 0, 1, dk);
    __syncthreads();  // the page before and its weights are no longer read (and qs is written)
    if (vec) {
      const int chunks = dk / 8;
      for (int i = tid; i < PTB_PAGE * chunks; i += THREADS) {
        const int j = i / chunks, e = (i % chunks) * 8;
        float f[8];
        if (j < valid) {
          unpack_bf16x8(*reinterpret_cast<const uint4*>(kp + size_t(j) * dk + e), f);
        } else {
#pragma unroll
          for (int u = 0; u < 8; ++u) f[u] = 0.f;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) kv[j * kstride + e + u] = f[u];
      }
    } else {
      for (int i = tid; i < PTB_PAGE * dk; i += THREADS) {
        const int j = i / dk, e = i % dk;
        kv[j * kstride + e] = (j < valid) ? to_f(kp[i]) : 0.f;
      }
    }
    __syncthreads();
    // scores: this thread owns keys j = c + 8 jj of row r
    float s[8];
#pragma unroll
    for (int jj = 0; jj < 8; ++jj) s[jj] = 0.f;
    const float* qr = qs + r * qstride;
    for (int e = 0; e < dk; ++e) {
      const float qe = qr[e];
#pragma unroll
      for (int jj = 0; jj < 8; ++jj) s[jj] = fmaf(qe, kv[(c + 8 * jj) * kstride + e], s[jj]);
    }
    float m_blk = -INFINITY;
#pragma unroll
    for (int jj = 0; jj < 8; ++jj) {
      const int key_pos = kb * PTB_PAGE + c + 8 * jj;
      s[jj] = (key_pos <= my_pos) ? s[jj] * scale : -INFINITY;
      m_blk = fmaxf(m_blk, s[jj]);
    }
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) m_blk = fmaxf(m_blk, __shfl_xor_sync(0xffffffffu, m_blk, o));
    const float m_new = fmaxf(m_run, m_blk);
    float corr = 1.f, l_blk = 0.f;
    if (m_new == -INFINITY) {
#pragma unroll
      for (int jj = 0; jj < 8; ++jj) ps[r * PTB_PAGE + c + 8 * jj] = 0.f;
    } else {
      corr = (m_run == -INFINITY) ? 0.f : expf(m_run - m_new);
#pragma unroll
      for (int jj = 0; jj < 8; ++jj) {
        const float p = (s[jj] == -INFINITY) ? 0.f : expf(s[jj] - m_new);
        ps[r * PTB_PAGE + c + 8 * jj] = p;
        l_blk += p;
      }
    }
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) l_blk += __shfl_xor_sync(0xffffffffu, l_blk, o);
    l_run = l_run * corr + l_blk;
    m_run = m_new;
    __syncwarp();  // a row's weights are written and read by the 8 threads of one warp
#pragma unroll
    for (int i = 0; i < DPT; ++i) acc[i] *= corr;
    for (int j = 0; j < PTB_PAGE; ++j) {
      const float p = ps[r * PTB_PAGE + j];
      const float* vr = kv + j * kstride;
#pragma unroll
      for (int i = 0; i < DPT; ++i) {
        const int e = c + 8 * i;
        if (e < rank) acc[i] = fmaf(p, vr[e], acc[i]);
      }
    }
  }
  if (n_splits > 1) {
    float* p = part + ((size_t(tile) * gridDim.y + blockIdx.y) * n_splits + split) * ROWS * size_t(rank + 2) +
               size_t(r) * (rank + 2);
    if (c == 0) {
      p[0] = m_run;
      p[1] = l_run;
    }
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
      const int e = c + 8 * i;
      if (e < rank) p[2 + e] = acc[i];
    }
    return;
  }
  if (my_row) {
    const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
    T* o = out + (size_t(start + q0 + my_tok) * heads + my_head) * rank;
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
      const int e = c + 8 * i;
      if (e < rank) o[e] = from_f<T>(acc[i] * inv);
    }
  }
}

// merges the splits of a tile in ascending order of their pages: one block per (tile, head chunk, row)
template <typename T>
__global__ void latent_join_kernel(const float* __restrict__ part, T* __restrict__ out, StepBatch sb,
                                   const int* __restrict__ tile_seq, const int* __restrict__ tile_q0, int heads,
                                   int rank, int tile_tokens, int heads_per_block, int n_splits) {
  extern __shared__ float jw[];   // the splits' weights exp(m_s - m) / l
  const int tile = blockIdx.x, h0 = blockIdx.y * heads_per_block, r = blockIdx.z;
  const int seq = tile_seq[tile], q0 = tile_q0[tile];
  const int toks = min(tile_tokens, sb.seq_new[seq] - q0), start = sb.seq_start[seq];
  const int ti = r / heads_per_block, hh = h0 + r % heads_per_block;
  if (!(ti < toks && hh < heads && r < tile_tokens * heads_per_block)) return;
  const float* base = part + (size_t(tile) * gridDim.y + blockIdx.y) * n_splits * ROWS * size_t(rank + 2) + size_t(r) * (rank + 2);
  const size_t split_stride = size_t(ROWS) * (rank + 2);
  if (threadIdx.x < 32) {
    float m = -INFINITY;
    for (int s = threadIdx.x; s < n_splits; s += 32) m = fmaxf(m, base[s * split_stride]);
    m = warp_max(m);
    float l = 0.f;
    for (int s = 0; s < n_splits; ++s) {      // ascending order, the same in every lane
      const float ms = base[s * split_stride];
      const float w = (ms == -INFINITY) ? 0.f : expf(ms - m);
      l += base[s * split_stride + 1] * w;
      if (threadIdx.x == 0) jw[s] = w;
    }
    __syncwarp();
    const float inv = l > 0.f ? 1.f / l : 0.f;
    for (int s = threadIdx.x; s < n_splits; s += 32) jw[s] *= inv;
  }
  __syncthreads();
  T* o = out + (size_t(start + q0 + ti) * heads + hh) * rank;
  for (int e = threadIdx.x; e < rank; e += blockDim.x) {
    float v = 0.f;
    for (int s = 0; s < n_splits; ++s) v = fmaf(base[s * split_stride + 2 + e], jw[s], v);
    o[e] = from_f<T>(v);
  }
}

template <typename T, int DPT>
int launch_latent(const float* q_abs, const void* q, int q_dim, int q_rot_off, const void* pool, float* part,
                  void* out, const StepBatch& sb, const int* tile_seq, const int* tile_q0, int n_tiles,
                  const float* rope_cos, const float* rope_sin, int rot_pairs, int interleaved, int heads, int rank,
                  int rot_dim, int tile_tokens, int heads_per_block, float scale, int n_splits, cudaStream_t stream) {
  const int dk = rank + rot_dim;
  const size_t smem = sizeof(float) * (size_t(ROWS) * (dk + 1) + size_t(PTB_PAGE) * (dk + 1) + ROWS * PTB_PAGE);
  if (smem > 220 * 1024) return PTB_ERR_SIZE;
  static size_t configured = 48 * 1024;
  if (smem > configured) {
    if (cudaFuncSetAttribute(latent_attention_kernel<T, DPT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             int(smem)) != cudaSuccess)
      return PTB_ERR_LAUNCH;
    configured = smem;
  }
  const int chunks = (heads + heads_per_block - 1) / heads_per_block;
  dim3 grid(n_tiles, chunks, n_splits);
  latent_attention_kernel<T, DPT><<<grid, THREADS, smem, stream>>>(
      q_abs, (const T*)q, q_dim, q_rot_off, (const T*)pool, part, (T*)out, sb, tile_seq, tile_q0, rope_cos, rope_sin,
      rot_pairs, interleaved, heads, rank, rot_dim, tile_tokens, heads_per_block, scale, n_splits);
  int rc = launch_status();
  if (rc != PTB_OK || n_splits <= 1) return rc;
  latent_join_kernel<T><<<dim3(n_tiles, chunks, ROWS), 128, n_splits * sizeof(float), stream>>>(
      part, (T*)out, sb, tile_seq, tile_q0, heads, rank, tile_tokens, heads_per_block, n_splits);
  return launch_status();
}

template <typename T>
int dispatch_latent(const float* q_abs, const void* q, int q_dim, int q_rot_off, const void* pool, float* part,
                    void* out, const StepBatch& sb, const int* tile_seq, const int* tile_q0, int n_tiles,
                    const float* rope_cos, const float* rope_sin, int rot_pairs, int interleaved, int heads, int rank,
                    int rot_dim, int tile_tokens, int heads_per_block, float scale, int n_splits,
                    cudaStream_t stream) {
#define PTB_LATENT(D)                                                                                             \
  return launch_latent<T, D>(q_abs, q, q_dim, q_rot_off, pool, part, out, sb, tile_seq, tile_q0, n_tiles, rope_cos, \
                             rope_sin, rot_pairs, interleaved, heads, rank, rot_dim, tile_tokens, heads_per_block,  \
                             scale, n_splits, stream)
  if (rank <= 64) PTB_LATENT(8);
  if (rank <= 128) PTB_LATENT(16);
  if (rank <= 256) PTB_LATENT(32);
  PTB_LATENT(64);
#undef PTB_LATENT
}

}  // namespace

PTB_API int ptb_latent_rows() { return ROWS; }

// float32 values of workspace that ptb_latent_attention needs with n_splits > 1
PTB_API long long ptb_latent_part_floats(int n_tiles, int heads, int heads_per_block, int n_splits, int rank) {
  if (n_splits <= 1) return 0;
  const long long chunks = (heads + heads_per_block - 1) / heads_per_block;
  return (long long)n_tiles * chunks * n_splits * ROWS * (rank + 2);
}

PTB_API int ptb_latent_store(int dtype, const void* src, long long src_stride, const float* norm_w, float eps,
                             void* pool, const StepBatch* sb, const float* rope_cos, const float* rope_sin,
                             int rot_pairs, int interleaved, int rank, int rot_dim, cudaStream_t stream) {
  if (sb->n_tokens <= 0) return PTB_OK;
  if (rank <= 0 || rot_dim < 0 || rot_pairs < 0 || 2 * rot_pairs > rot_dim) return PTB_ERR_SIZE;
  if (rot_pairs > 0 && (rope_cos == nullptr || rope_sin == nullptr)) return PTB_ERR_SIZE;
  if (dtype == PTB_F32)
    latent_store_kernel<float><<<sb->n_tokens, 128, 0, stream>>>((const float*)src, src_stride, norm_w, eps,
                                                                 (float*)pool, *sb, rope_cos, rope_sin, rot_pairs,
                                                                 interleaved, rank, rot_dim);
  else if (dtype == PTB_BF16)
    latent_store_kernel<__nv_bfloat16><<<sb->n_tokens, 128, 0, stream>>>(
        (const __nv_bfloat16*)src, src_stride, norm_w, eps, (__nv_bfloat16*)pool, *sb, rope_cos, rope_sin, rot_pairs,
        interleaved, rank, rot_dim);
  else
    return PTB_ERR_DTYPE;
  return launch_status();
}

PTB_API int ptb_latent_attention(int dtype, const float* q_abs, const void* q, int q_dim, int q_rot_off,
                                 const void* pool, float* part, void* out, const StepBatch* sb, const int* tile_seq,
                                 const int* tile_q0, int n_tiles, const float* rope_cos, const float* rope_sin,
                                 int rot_pairs, int interleaved, int heads, int rank, int rot_dim, int tile_tokens,
                                 int heads_per_block, float scale, int n_splits, cudaStream_t stream) {
  if (n_tiles <= 0) return PTB_OK;
  if (heads <= 0 || rank <= 0 || rank > 512 || rot_dim < 0 || rot_pairs < 0 || 2 * rot_pairs > rot_dim ||
      tile_tokens <= 0 || heads_per_block <= 0 || tile_tokens * heads_per_block > ROWS || n_splits < 1 ||
      n_splits > 65535 || (heads + heads_per_block - 1) / heads_per_block > 65535)
    return PTB_ERR_SIZE;
  if (n_splits > 1 && part == nullptr) return PTB_ERR_SIZE;
  if (rot_pairs > 0 && (rope_cos == nullptr || rope_sin == nullptr)) return PTB_ERR_SIZE;
  if (dtype == PTB_F32)
    return dispatch_latent<float>(q_abs, q, q_dim, q_rot_off, pool, part, out, *sb, tile_seq, tile_q0, n_tiles,
                                  rope_cos, rope_sin, rot_pairs, interleaved, heads, rank, rot_dim, tile_tokens,
                                  heads_per_block, scale, n_splits, stream);
  if (dtype == PTB_BF16)
    return dispatch_latent<__nv_bfloat16>(q_abs, q, q_dim, q_rot_off, pool, part, out, *sb, tile_seq, tile_q0, n_tiles,
                                          rope_cos, rope_sin, rot_pairs, interleaved, heads, rank, rot_dim,
                                          tile_tokens, heads_per_block, scale, n_splits, stream);
  return PTB_ERR_DTYPE;
}

// ------------------------------------------------------------------------------------------------
// The same attention in bfloat16 on the tensor cores (mma.m16n8k16, float32 sums), for rank a multiple
// of 64 and rot_dim a multiple of 16. A block of 4 warps takes the 16 rows of a tile (the heads of a
// token in a step of single tokens) and walks its share of the key pages. A page [64][rank + rot_dim]
// comes into shared memory once (cp.async, rows 16 bytes apart from a multiple of 128 so that ldmatrix
// meets no bank twice) and serves both products, for up to four groups of 4 warps with 16 rows each (a tile of a
// prompt is 16 tokens x 4 heads, so that a staged page meets 64 rows): warp w of a group forms the scores of keys 16 w .. 16 w + 15
// (S = Q K^T over all rank + rot_dim entries), the warps exchange row maxima and sums through shared
// memory, the weights go to shared memory as bfloat16, and warp w adds P V for the columns
// w rank / 4 .. (w + 1) rank / 4 of the output, V being the first `rank` entries of the same rows.
// The query rows are rounded to bfloat16 once (q_abs comes in float32); scores, maxima, sums and the
// output sums are float32. Splits and their join are those of the general kernel.
#include "mma_common.cuh"

namespace {

constexpr int MTHREADS = 128;

// NF: 8-column fragments of the output per warp (rank = 32 NF). TG: groups of 4 warps; every group has 16
// rows of the tile (a tile of a prompt holds 16 TG rows: tokens x heads), and all groups use one staged page.
template <int NF, int TG>
__global__ void __launch_bounds__(MTHREADS * TG)
latent_attention_mma_kernel(const float* __restrict__ q_abs, const __nv_bfloat16* __restrict__ q, int q_dim,
                            int q_rot_off, const __nv_bfloat16* __restrict__ pool, float* __restrict__ part,
                            __nv_bfloat16* __restrict__ out, StepBatch sb, const int* __restrict__ tile_seq,
                            const int* __restrict__ tile_q0, const float* __restrict__ rope_cos,
                            const float* __restrict__ rope_sin, int rot_pairs, int interleaved, int heads, int rank,
                            int rot_dim, int tile_tokens, int heads_per_block, float scale, int n_splits) {
  extern __shared__ __align__(128) unsigned char msm[];
  constexpr int NT = MTHREADS * TG, QROWS = ROWS * TG;
  const int dk = rank + rot_dim;
  const int rowb = dk * 2 + 16;                       // bytes of a staged row
  unsigned char* q_s = msm;                           // [16 TG][rowb]
  unsigned char* k_s = q_s + QROWS * rowb;            // [64][rowb]
  unsigned char* p_all = k_s + PTB_PAGE * rowb;       // [TG][16][144]: 64 weights and 16 bytes of padding a row
  float* wmax_all = reinterpret_cast<float*>(p_all + TG * 16 * 144);   // [TG][4][16]
  float* wsum_all = wmax_all + TG * 64;                                 // [TG][4][16]

  const int tile = blockIdx.x, h0 = blockIdx.y * heads_per_block, split = blockIdx.z;
  const int seq = tile_seq[tile], q0 = tile_q0[tile];
  const int n_new = sb.seq_new[seq], past = sb.seq_past[seq], start = sb.seq_start[seq];
  const int toks = min(tile_tokens, n_new - q0);
  const int tid = threadIdx.x, lane = tid % 32;
  const int tg = tid / MTHREADS, warp = (tid / 32) % 4;      // group of warps, warp in the group
  const int used_rows = tile_tokens * heads_per_block;
  unsigned char* p_s = p_all + tg * 16 * 144;
  float* wmax = wmax_all + tg * 64;
  float* wsum = wsum_all + tg * 64;

  // the query rows, rounded to bfloat16: [q_abs | rotated part]
  for (int i = tid; i < QROWS * rank; i += NT) {
    const int rr = i / rank, e = i % rank;
    const int ti = rr / heads_per_block, hh = h0 + rr % heads_per_block;
    const bool ok = ti < toks && hh < heads && rr < used_rows;
    const float v = ok ? q_abs[(size_t(start + q0 + ti) * heads + hh) * rank + e] : 0.f;
    reinterpret_cast<__nv_bfloat16*>(q_s + rr * rowb)[e] = __float2bfloat16_rn(v);
  }
  const int items = rot_pairs + (rot_dim - 2 * rot_pairs);
  for (int i = tid; i < QROWS * items; i += NT) {
    const int rr = i / items, e = i % items;
    const int ti = rr / heads_per_block, hh = h0 + rr % heads_per_block;
    const bool ok = ti < toks && hh < heads && rr < used_rows;
    const size_t tok = size_t(start + q0 + ti);
    const __nv_bfloat16* src = q + (tok * heads + hh) * q_dim + q_rot_off;
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(q_s + rr * rowb) + rank;
    if (e < rot_pairs) {
      const int ia = interleaved ? 2 * e : e, ib = interleaved ? 2 * e + 1 : e + rot_pairs;
      float a = 0.f, b = 0.f;
      if (ok) rotate_pair(to_f(src[ia]), to_f(src[ib]), rope_cos[tok * rot_pairs + e], rope_sin[tok * rot_pairs + e], a, b);
      dst[ia] = __float2bfloat16_rn(a);
      dst[ib] = __float2bfloat16_rn(b);
    } else {
      const int j = 2 * rot_pairs + (e - rot_pairs);
      dst[j] = ok ? src[j] : __float2bfloat16_rn(0.f);
    }
  }

  // this thread's two rows of its group's 16 (accumulator layout of mma.m16n8k16)
  const int r_lo = lane / 4, r_hi = r_lo + 8;
  int pos_of[2];
#pragma unroll
  for (int hf = 0; hf < 2; ++hf) {
    const int rr = tg * 16 + (hf ? r_hi : r_lo);
    const int ti = rr / heads_per_block, hh = h0 + rr % heads_per_block;
    pos_of[hf] = (ti < toks && hh < heads && rr < used_rows) ? past + q0 + ti : -1;
  }
  float acc[NF][4];
#pragma unroll
  for (int j = 0; j < NF; ++j)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[j][c] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

  const int last_pos = past + q0 + toks - 1;
  const int n_blocks = last_pos / PTB_PAGE + 1;
  const int per = (n_blocks + n_splits - 1) / n_splits;
  const int kb_lo = split * per, kb_hi = min(n_blocks, kb_lo + per) - 1;
  const int* pages = sb.pages + size_t(seq) * sb.pages_stride;
  const int chunks = dk / 8;
  const uint32_t q_base = smem_u32(q_s) + tg * 16 * rowb, k_base = smem_u32(k_s), p_base = smem_u32(p_s);
  const int col0 = warp * NF * 8;       // first output column of this warp

  for (int kb = kb_lo; kb <= kb_hi; ++kb) {
    const __nv_bfloat16* kp = pool + kv_offset(pages[kb], 0, 0, 1, dk);
    __syncthreads();   // the page before is no longer read (and the query rows are written)
    for (int i = tid; i < PTB_PAGE * chunks; i += NT) {
      const int j = i / chunks, c = i % chunks;
      cp_async16(k_base + j * rowb + c * 16, kp + size_t(j) * dk + c * 8);
    }
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();
    // scores of keys 16 warp .. 16 warp + 15
    float s[2][4];
#pragma unroll
    for (int f = 0; f < 2; ++f)
#pragma unroll
      for (int c = 0; c < 4; ++c) s[f][c] = 0.f;
    for (int ks = 0; ks < dk / 16; ++ks) {
      uint32_t a[4], b0, b1, b2, b3;
      ldmatrix_x4(a[0], a[1], a[2], a[3], q_base + (lane & 15) * rowb + (ks * 2 + (lane >> 4)) * 16);
      const int id = lane >> 3;
      ldmatrix_x4(b0, b1, b2, b3, k_base + (warp * 16 + (id >> 1) * 8 + (lane & 7)) * rowb + (ks * 2 + (id & 1)) * 16);
      mma_bf16(s[0], a, b0, b1);
      mma_bf16(s[1], a, b2, b3);
    }
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int f = 0; f < 2; ++f)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int key_pos = kb * PTB_PAGE + warp * 16 + f * 8 + (lane % 4) * 2 + (c & 1);
        const int hf = c >> 1;
        s[f][c] = (key_pos <= pos_of[hf]) ? s[f][c] * scale : -INFINITY;
        mx[hf] = fmaxf(mx[hf], s[f][c]);
      }
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      mx[hf] = fmaxf(mx[hf], __shfl_xor_sync(0xffffffffu, mx[hf], 1));
      mx[hf] = fmaxf(mx[hf], __shfl_xor_sync(0xffffffffu, mx[hf], 2));
    }
    if (lane % 4 == 0) {
      wmax[warp * 16 + r_lo] = mx[0];
      wmax[warp * 16 + r_hi] = mx[1];
    }
    __syncthreads();
    float corr[2], m_new[2], sum[2] = {0.f, 0.f};
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      const int rr = hf ? r_hi : r_lo;
      const float mb = fmaxf(fmaxf(wmax[rr], wmax[16 + rr]), fmaxf(wmax[32 + rr], wmax[48 + rr]));
      m_new[hf] = fmaxf(m_run[hf], mb);
      corr[hf] = (m_run[hf] == -INFINITY) ? 0.f : expf(m_run[hf] - m_new[hf]);
      if (m_new[hf] == -INFINITY) corr[hf] = 1.f;      // nothing seen yet: the sums stay 0
    }
#pragma unroll
    for (int f = 0; f < 2; ++f)
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const float p0 = (s[f][hf * 2] == -INFINITY) ? 0.f : expf(s[f][hf * 2] - m_new[hf]);
        const float p1 = (s[f][hf * 2 + 1] == -INFINITY) ? 0.f : expf(s[f][hf * 2 + 1] - m_new[hf]);
        // the weights as the second product sees them, and their sum from the same rounded values
        const __nv_bfloat162 pr = __floats2bfloat162_rn(p0, p1);
        sum[hf] += __bfloat162float(pr.x) + __bfloat162float(pr.y);
        const int rr = hf ? r_hi : r_lo;
        *reinterpret_cast<__nv_bfloat162*>(p_s + rr * 144 + (warp * 16 + f * 8 + (lane % 4) * 2) * 2) = pr;
      }
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      sum[hf] += __shfl_xor_sync(0xffffffffu, sum[hf], 1);
      sum[hf] += __shfl_xor_sync(0xffffffffu, sum[hf], 2);
    }
    if (lane % 4 == 0) {
      wsum[warp * 16 + r_lo] = sum[0];
      wsum[warp * 16 + r_hi] = sum[1];
    }
    __syncthreads();
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      const int rr = hf ? r_hi : r_lo;
      l_run[hf] = l_run[hf] * corr[hf] + ((wsum[rr] + wsum[16 + rr]) + (wsum[32 + rr] + wsum[48 + rr]));
      m_run[hf] = m_new[hf];
    }
#pragma unroll
    for (int j = 0; j < NF; ++j) {
      acc[j][0] *= corr[0];
      acc[j][1] *= corr[0];
      acc[j][2] *= corr[1];
      acc[j][3] *= corr[1];
    }
    // O += P V for this warp's columns
#pragma unroll
    for (int ks = 0; ks < PTB_PAGE / 16; ++ks) {
      uint32_t a[4];
      ldmatrix_x4(a[0], a[1], a[2], a[3], p_base + (lane & 15) * 144 + (ks * 2 + (lane >> 4)) * 16);
      const int id = lane >> 3;
#pragma unroll
      for (int jp = 0; jp < NF / 2; ++jp) {
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(b0, b1, b2, b3,
                          k_base + (ks * 16 + (id & 1) * 8 + (lane & 7)) * rowb + (col0 + jp * 16 + (id >> 1) * 8) * 2);
        mma_bf16(acc[2 * jp], a, b0, b1);
        mma_bf16(acc[2 * jp + 1], a, b2, b3);
      }
    }
  }
  const int c0 = (lane % 4) * 2;
#pragma unroll
  for (int hf = 0; hf < 2; ++hf) {
    const int rl = hf ? r_hi : r_lo, rr = tg * 16 + rl;
    if (n_splits > 1) {      // only with TG = 1
      float* p = part + ((size_t(tile) * gridDim.y + blockIdx.y) * n_splits + split) * ROWS * size_t(rank + 2) +
                 size_t(rl) * (rank + 2);
      if (warp == 0 && lane % 4 == 0) {
        p[0] = m_run[hf];
        p[1] = l_run[hf];
      }
#pragma unroll
      for (int j = 0; j < NF; ++j) {
        p[2 + col0 + j * 8 + c0] = acc[j][hf * 2];
        p[2 + col0 + j * 8 + c0 + 1] = acc[j][hf * 2 + 1];
      }
    } else if (pos_of[hf] >= 0) {
      const int ti = rr / heads_per_block, hh = h0 + rr % heads_per_block;
      const float inv = l_run[hf] > 0.f ? 1.f / l_run[hf] : 0.f;
      __nv_bfloat16* o = out + (size_t(start + q0 + ti) * heads + hh) * rank + col0;
#pragma unroll
      for (int j = 0; j < NF; ++j)
        *reinterpret_cast<__nv_bfloat162*>(o + j * 8 + c0) = __floats2bfloat162_rn(acc[j][hf * 2] * inv, acc[j][hf * 2 + 1] * inv);
    }
  }
}

template <int NF, int TG>
int launch_latent_mma_tg(const float* q_abs, const void* q, int q_dim, int q_rot_off, const void* pool, float* part,
                         void* out, const StepBatch& sb, const int* tile_seq, const int* tile_q0, int n_tiles,
                         const float* rope_cos, const float* rope_sin, int rot_pairs, int interleaved, int heads, int rank,
                         int rot_dim, int tile_tokens, int heads_per_block, float scale, int n_splits, cudaStream_t stream) {
  const int rowb = (rank + rot_dim) * 2 + 16;
  const size_t smem = size_t(16 * TG + PTB_PAGE) * rowb + TG * (16 * 144 + 2 * 64 * sizeof(float));
  if (smem > 220 * 1024) return PTB_ERR_SIZE;
  static size_t configured = 48 * 1024;
  if (smem > configured) {
    if (cudaFuncSetAttribute(latent_attention_mma_kernel<NF, TG>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) !=
        cudaSuccess)
      return PTB_ERR_LAUNCH;
    configured = smem;
  }
  const int chunks = (heads + heads_per_block - 1) / heads_per_block;
  latent_attention_mma_kernel<NF, TG><<<dim3(n_tiles, chunks, n_splits), MTHREADS * TG, smem, stream>>>(
      q_abs, (const __nv_bfloat16*)q, q_dim, q_rot_off, (const __nv_bfloat16*)pool, part, (__nv_bfloat16*)out, sb,
      tile_seq, tile_q0, rope_cos, rope_sin, rot_pairs, interleaved, heads, rank, rot_dim, tile_tokens, heads_per_block,
      scale, n_splits);
  int rc = launch_status();
  if (rc != PTB_OK || n_splits <= 1) return rc;
  latent_join_kernel<__nv_bfloat16><<<dim3(n_tiles, chunks, ROWS), 128, n_splits * sizeof(float), stream>>>(
      part, (__nv_bfloat16*)out, sb, tile_seq, tile_q0, heads, rank, tile_tokens, heads_per_block, n_splits);
  return launch_status();
}

template <int NF>
int launch_latent_mma(const float* q_abs, const void* q, int q_dim, int q_rot_off, const void* pool, float* part,
                      void* out, const StepBatch& sb, const int* tile_seq, const int* tile_q0, int n_tiles,
                      const float* rope_cos, const float* rope_sin, int rot_pairs, int interleaved, int heads, int rank,
                      int rot_dim, int tile_tokens, int heads_per_block, float scale, int n_splits, cudaStream_t stream) {
  const int rows = tile_tokens * heads_per_block;
#define PTB_LTG(TGV)                                                                                                  \
  return launch_latent_mma_tg<NF, TGV>(q_abs, q, q_dim, q_rot_off, pool, part, out, sb, tile_seq, tile_q0, n_tiles,     \
                                       rope_cos, rope_sin, rot_pairs, interleaved, heads, rank, rot_dim, tile_tokens,   \
                                       heads_per_block, scale, n_splits, stream)
  if (rows <= 16) PTB_LTG(1);
  if (n_splits != 1) return PTB_ERR_SIZE;
  if (rows <= 32) PTB_LTG(2);
  PTB_LTG(4);
#undef PTB_LTG
}

}  // namespace

PTB_API int ptb_latent_attention_mma_supports(int rank, int rot_dim) {
  return rank > 0 && rank <= 512 && rank % 64 == 0 && rot_dim >= 0 && rot_dim % 16 == 0;
}

PTB_API int ptb_latent_attention_mma(const float* q_abs, const void* q, int q_dim, int q_rot_off, const void* pool,
                                     float* part, void* out, const StepBatch* sb, const int* tile_seq,
                                     const int* tile_q0, int n_tiles, const float* rope_cos, const float* rope_sin,
                                     int rot_pairs, int interleaved, int heads, int rank, int rot_dim, int tile_tokens,
                                     int heads_per_block, float scale, int n_splits, cudaStream_t stream) {
  if (n_tiles <= 0) return PTB_OK;
  if (!ptb_latent_attention_mma_supports(rank, rot_dim) || heads <= 0 || rot_pairs < 0 || 2 * rot_pairs > rot_dim ||
      tile_tokens <= 0 || heads_per_block <= 0 || tile_tokens * heads_per_block > 4 * ROWS || n_splits < 1 ||
      n_splits > 65535 || (heads + heads_per_block - 1) / heads_per_block > 65535)
    return PTB_ERR_SIZE;
  if (n_splits > 1 && part == nullptr) return PTB_ERR_SIZE;
  if (rot_pairs > 0 && (rope_cos == nullptr || rope_sin == nullptr)) return PTB_ERR_SIZE;
  if (!aligned16(pool) || !aligned16(out)) return PTB_ERR_ALIGN;
#define PTB_LMMA(NFV)                                                                                               \
  return launch_latent_mma<NFV>(q_abs, q, q_dim, q_rot_off, pool, part, out, *sb, tile_seq, tile_q0, n_tiles, rope_cos, \
                                rope_sin, rot_pairs, interleaved, heads, rank, rot_dim, tile_tokens, heads_per_block,   \
                                scale, n_splits, stream)
  switch (rank / 64) {
    case 1: PTB_LMMA(2);
    case 2: PTB_LMMA(4);
    case 3: PTB_LMMA(6);
    case 4: PTB_LMMA(8);
    case 5: PTB_LMMA(10);
    case 6: PTB_LMMA(12);
    case 7: PTB_LMMA(14);
    default: PTB_LMMA(16);
  }
#undef PTB_LMMA
}

// ------------------------------------------------------------------------------------------------
// Prompts in bfloat16 with per-head sizes that the tcgen05 prompt kernel takes (csrc/attention_tc.cu: 64 or
// 128): the cached latents of the step's sequences are unfolded into per-head keys [W_uk[h] c | kr | 0] and
// values [W_uv[h] c | 0] in scratch pools laid out like a cache entry's ([pages][heads][64][hd], the same
// page numbers), and that kernel runs on them. The pieces here: the context's cache rows gathered into
// dense matrices (for the library's product with [W_uk; W_uv]), the product's rows scattered into the
// pools, the queries laid out as [plain | rotated | 0], and the output gate on the heads' first vdim entries.
namespace {

__global__ void latent_gather_kernel(const __nv_bfloat16* __restrict__ pool, StepBatch sb,
                                     const int* __restrict__ ctx_seq, const int* __restrict__ ctx_pos,
                                     __nv_bfloat16* __restrict__ c_rows, __nv_bfloat16* __restrict__ kr_rows, int rank,
                                     int rot_dim) {
  const int i = blockIdx.x, seq = ctx_seq[i], pos = ctx_pos[i];
  const int page = sb.pages[size_t(seq) * sb.pages_stride + pos / PTB_PAGE];
  const __nv_bfloat16* src = pool + kv_offset(page, 0, pos % PTB_PAGE, 1, rank + rot_dim);
  for (int e = threadIdx.x; e < rank; e += blockDim.x) c_rows[size_t(i) * rank + e] = src[e];
  for (int e = threadIdx.x; e < rot_dim; e += blockDim.x) kr_rows[size_t(i) * rot_dim + e] = src[rank + e];
}

// kv [ctx, heads * dim + heads * vdim]: a context row's keys of all heads, then its values of all heads
__global__ void latent_unfold_kernel(const __nv_bfloat16* __restrict__ kv, const __nv_bfloat16* __restrict__ kr_rows,
                                     StepBatch sb, const int* __restrict__ ctx_seq, const int* __restrict__ ctx_pos,
                                     __nv_bfloat16* __restrict__ k_tmp, __nv_bfloat16* __restrict__ v_tmp, int heads,
                                     int dim, int rot_dim, int vdim, int hd) {
  const int i = blockIdx.x, seq = ctx_seq[i], pos = ctx_pos[i];
  const int page = sb.pages[size_t(seq) * sb.pages_stride + pos / PTB_PAGE], slot = pos % PTB_PAGE;
  const size_t width = size_t(heads) * (dim + vdim);
  const __nv_bfloat16* row = kv + size_t(i) * width;
  const int dq = dim + rot_dim;
  for (int idx = threadIdx.x; idx < heads * dq; idx += blockDim.x) {
    const int h = idx / dq, e = idx % dq;
    k_tmp[kv_offset(page, h, slot, heads, hd) + e] = (e < dim) ? row[size_t(h) * dim + e] : kr_rows[size_t(i) * rot_dim + (e - dim)];
  }
  for (int idx = threadIdx.x; idx < heads * vdim; idx += blockDim.x) {
    const int h = idx / vdim, e = idx % vdim;
    v_tmp[kv_offset(page, h, slot, heads, hd) + e] = row[size_t(heads) * dim + size_t(h) * vdim + e];
  }
}

__global__ void latent_q_unfold_kernel(const __nv_bfloat16* __restrict__ q, const float* __restrict__ rope_cos,
                                       const float* __restrict__ rope_sin, int rot_pairs, int interleaved,
                                       __nv_bfloat16* __restrict__ out, int heads, int dim, int rot_dim, int hd) {
  const size_t t = blockIdx.x;
  const int dq = dim + rot_dim;
  const int items = dim + rot_pairs + (rot_dim - 2 * rot_pairs) + (hd - dq);     // per head: plain, pairs, unrotated rest, padding
  for (int idx = threadIdx.x; idx < heads * items; idx += blockDim.x) {
    const int h = idx / items;
    int e = idx % items;
    const __nv_bfloat16* src = q + (t * heads + h) * dq;
    __nv_bfloat16* dst = out + (t * heads + h) * hd;
    if (e < dim) { dst[e] = src[e]; continue; }
    e -= dim;
    if (e < rot_pairs) {
      const int ia = interleaved ? 2 * e : e, ib = interleaved ? 2 * e + 1 : e + rot_pairs;
      float a, b;
      rotate_pair(to_f(src[dim + ia]), to_f(src[dim + ib]), rope_cos[t * rot_pairs + e], rope_sin[t * rot_pairs + e], a, b);
      dst[dim + ia] = __float2bfloat16_rn(a);
      dst[dim + ib] = __float2bfloat16_rn(b);
      continue;
    }
    e -= rot_pairs;
    if (e < rot_dim - 2 * rot_pairs) { dst[dim + 2 * rot_pairs + e] = src[dim + 2 * rot_pairs + e]; continue; }
    e -= rot_dim - 2 * rot_pairs;
    dst[dq + e] = __float2bfloat16_rn(0.f);
  }
}

// out[t, h, :vdim] = o[t, h, :vdim] * sigmoid(gate[t, h, :vdim]); o rows are hd wide
__global__ void gate_heads_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ gate,
                                  long long gate_t, __nv_bfloat16* __restrict__ out, long long total, int heads, int vdim,
                                  int hd) {
  const size_t stride = size_t(gridDim.x) * blockDim.x;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < size_t(total); i += stride) {
    const int e = int(i % vdim), h = int((i / vdim) % heads);
    const size_t t = i / (size_t(vdim) * heads);
    const float g = to_f(gate[t * gate_t + size_t(h) * vdim + e]);
    out[i] = __float2bfloat16_rn(to_f(o[(t * heads + h) * hd + e]) / (1.f + expf(-g)));
  }
}

}  // namespace

PTB_API int ptb_latent_gather(const void* pool, const StepBatch* sb, const int* ctx_seq, const int* ctx_pos, int n_ctx,
                              void* c_rows, void* kr_rows, int rank, int rot_dim, cudaStream_t stream) {
  if (n_ctx <= 0) return PTB_OK;
  if (rank <= 0 || rot_dim < 0) return PTB_ERR_SIZE;
  latent_gather_kernel<<<n_ctx, 128, 0, stream>>>((const __nv_bfloat16*)pool, *sb, ctx_seq, ctx_pos, (__nv_bfloat16*)c_rows,
                                                  (__nv_bfloat16*)kr_rows, rank, rot_dim);
  return launch_status();
}

PTB_API int ptb_latent_unfold(const void* kv, const void* kr_rows, const StepBatch* sb, const int* ctx_seq,
                              const int* ctx_pos, int n_ctx, void* k_tmp, void* v_tmp, int heads, int dim, int rot_dim,
                              int vdim, int hd, cudaStream_t stream) {
  if (n_ctx <= 0) return PTB_OK;
  if (heads <= 0 || dim <= 0 || rot_dim < 0 || vdim <= 0 || dim + rot_dim > hd || vdim > hd) return PTB_ERR_SIZE;
  latent_unfold_kernel<<<n_ctx, 256, 0, stream>>>((const __nv_bfloat16*)kv, (const __nv_bfloat16*)kr_rows, *sb, ctx_seq,
                                                  ctx_pos, (__nv_bfloat16*)k_tmp, (__nv_bfloat16*)v_tmp, heads, dim, rot_dim,
                                                  vdim, hd);
  return launch_status();
}

PTB_API int ptb_latent_q_unfold(const void* q, const float* rope_cos, const float* rope_sin, int rot_pairs,
                                int interleaved, void* out, int n_tokens, int heads, int dim, int rot_dim, int hd,
                                cudaStream_t stream) {
  if (n_tokens <= 0) return PTB_OK;
  if (heads <= 0 || dim <= 0 || rot_dim < 0 || dim + rot_dim > hd || 2 * rot_pairs > rot_dim) return PTB_ERR_SIZE;
  if (rot_pairs > 0 && (rope_cos == nullptr || rope_sin == nullptr)) return PTB_ERR_SIZE;
  latent_q_unfold_kernel<<<n_tokens, 256, 0, stream>>>((const __nv_bfloat16*)q, rope_cos, rope_sin, rot_pairs, interleaved,
                                                       (__nv_bfloat16*)out, heads, dim, rot_dim, hd);
  return launch_status();
}

PTB_API int ptb_gate_heads(const void* o, const void* gate, long long gate_t, void* out, int n_tokens, int heads, int vdim,
                           int hd, cudaStream_t stream) {
  const long long total = (long long)n_tokens * heads * vdim;
  if (total <= 0) return PTB_OK;
  const size_t want = (size_t(total) + 255) / 256, most = size_t(sm_count()) * 16;
  gate_heads_kernel<<<int(want < most ? want : most), 256, 0, stream>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)gate,
                                                                       gate_t, (__nv_bfloat16*)out, total, heads, vdim, hd);
  return launch_status();
}
