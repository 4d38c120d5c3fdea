// Kernels for models whose residual stream is float32 while their matrices are bfloat16: the norm
// that reads the float32 stream and writes the model dtype, and the float32 sum of the stream with
// a branch's result (of either dtype).
#include "common.cuh"

namespace {

// y = norm(x [+ addend]) * gain [+ bias]; x, and the sum written to sum_out, are float32; addend is
// float32 or bfloat16 (TA); y is float32 or bfloat16 (TO). kind 0: LayerNorm (mean, then centred
// variance), kind 1: RMSNorm (x / sqrt(mean(x^2) + eps)). The row sits in shared memory as float32.
template <typename TA, typename TO>
__global__ void norm_stream_kernel(const float* __restrict__ x, const TA* __restrict__ addend,
                                   float* __restrict__ sum_out, const float* __restrict__ gain,
                                   const float* __restrict__ bias, TO* __restrict__ y, int width, float eps, int kind) {
  extern __shared__ float row[];
  __shared__ float scratch[32];
  const size_t base = size_t(blockIdx.x) * width;
  float s = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float v = x[base + i];
    if (addend) {
      v += to_f(addend[base + i]);
      sum_out[base + i] = v;
    }
    row[i] = v;
    s += v;
  }
  float mean = 0.f;
  if (kind == 0) mean = block_sum(s, scratch) / float(width);
  float q = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float c = row[i] - mean;
    q += c * c;
  }
  const float var = block_sum(q, scratch) / float(width);
  const float rstd = 1.0f / sqrtf(var + eps);
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float a = (row[i] - mean) * rstd * gain[i];
    if (bias) a += bias[i];
    y[base + i] = from_f<TO>(a);
  }
}

template <typename TA>
__global__ void add_stream_kernel(const float* __restrict__ x, const TA* __restrict__ a, float* __restrict__ out,
                                  size_t total) {
  const size_t stride = size_t(gridDim.x) * blockDim.x;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) out[i] = x[i] + to_f(a[i]);
}

// The closing norm of a branch and the stream's sum in one pass, optionally with the next sublayer's opening norm:
//     out = x + mult * (y / sqrt(mean(y^2) + eps)) * gain,        next = (out / sqrt(mean(out^2) + eps_next)) * gain_next.
// x and out are the float32 stream; y is the branch's result (TA: float32 or bfloat16); next (TO) is written only
// when gain_next is given. The row's y and sum sit in shared memory as float32.
template <typename TA, typename TO>
__global__ void post_norm_add_kernel(const float* __restrict__ x, const TA* __restrict__ y, const float* __restrict__ gain,
                                     float eps, float mult, float* __restrict__ out, const float* __restrict__ gain_next,
                                     float eps_next, TO* __restrict__ next, int width) {
  extern __shared__ float row[];
  __shared__ float scratch[32];
  const size_t base = size_t(blockIdx.x) * width;
  float q = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float v = to_f(y[base + i]);
    row[i] = v;
    q = fmaf(v, v, q);
  }
  const float rstd = 1.0f / sqrtf(block_sum(q, scratch) / float(width) + eps);
  float q2 = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float v = x[base + i] + mult * (row[i] * rstd * gain[i]);
    out[base + i] = v;
    row[i] = v;
    q2 = fmaf(v, v, q2);
  }
  if (gain_next == nullptr) return;
  const float rstd2 = 1.0f / sqrtf(block_sum(q2, scratch) / float(width) + eps_next);
  for (int i = threadIdx.x; i < width; i += blockDim.x) next[base + i] = from_f<TO>(row[i] * rstd2 * gain_next[i]);
}

// The stream's first value: out[t] = table[ids[t]] + positions[pos[t]] in float32 (a learned vector per position).
// An id or a position outside its table is clamped and bit 0 or bit 1 of *status is raised.
template <typename T>
__global__ void embed_sum_kernel(const int* __restrict__ ids, const int* __restrict__ pos, const T* __restrict__ table,
                                 const T* __restrict__ positions, float* __restrict__ out, int width, int rows,
                                 int pos_rows, int* __restrict__ status) {
  const size_t t = blockIdx.x;
  int id = ids[t], p = pos[t];
  if (id < 0 || id >= rows) {
    if (threadIdx.x == 0 && status) atomicOr(status, 1);
    id = min(max(id, 0), rows - 1);
  }
  if (p < 0 || p >= pos_rows) {
    if (threadIdx.x == 0 && status) atomicOr(status, 2);
    p = min(max(p, 0), pos_rows - 1);
  }
  const T* a = table + size_t(id) * width;
  const T* b = positions + size_t(p) * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) out[t * width + i] = to_f(a[i]) + to_f(b[i]);
}

template <typename TA, typename TO>
int launch_norm_stream(const float* x, const void* addend, float* sum_out, const float* gain, const float* bias,
                       void* y, int n, int width, float eps, int kind, cudaStream_t stream) {
  const size_t smem = size_t(width) * sizeof(float);
  static size_t configured = 48 * 1024;
  if (smem > configured) {
    if (cudaFuncSetAttribute(norm_stream_kernel<TA, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) !=
        cudaSuccess)
      return PTB_ERR_LAUNCH;
    configured = smem;
  }
  const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
  norm_stream_kernel<TA, TO><<<n, threads, smem, stream>>>(x, (const TA*)addend, sum_out, gain, bias, (TO*)y, width,
                                                           eps, kind);
  return launch_status();
}

}  // namespace

PTB_API int ptb_norm_stream(const float* x, int addend_dtype, const void* addend, float* sum_out, const float* gain,
                            const float* bias, int out_dtype, void* y, int n, int width, float eps, int kind,
                            cudaStream_t stream) {
  if (n <= 0) return PTB_OK;
  if (width <= 0 || kind < 0 || kind > 1 || size_t(width) * 4 > 200 * 1024) return PTB_ERR_SIZE;
  if ((addend == nullptr) != (sum_out == nullptr)) return PTB_ERR_SIZE;
  const bool a16 = addend != nullptr && addend_dtype == PTB_BF16;
  if (addend != nullptr && addend_dtype != PTB_BF16 && addend_dtype != PTB_F32) return PTB_ERR_DTYPE;
  if (out_dtype == PTB_F32)
    return a16 ? launch_norm_stream<__nv_bfloat16, float>(x, addend, sum_out, gain, bias, y, n, width, eps, kind, stream)
               : launch_norm_stream<float, float>(x, addend, sum_out, gain, bias, y, n, width, eps, kind, stream);
  if (out_dtype == PTB_BF16)
    return a16 ? launch_norm_stream<__nv_bfloat16, __nv_bfloat16>(x, addend, sum_out, gain, bias, y, n, width, eps,
                                                                  kind, stream)
               : launch_norm_stream<float, __nv_bfloat16>(x, addend, sum_out, gain, bias, y, n, width, eps, kind,
                                                          stream);
  return PTB_ERR_DTYPE;
}

// out = x + a with x and out float32 and a float32 or bfloat16
PTB_API int ptb_add_stream(const float* x, int a_dtype, const void* a, float* out, long long total,
                           cudaStream_t stream) {
  if (total <= 0) return PTB_OK;
  const int threads = 256;
  const size_t want = (size_t(total) + threads - 1) / threads, most = size_t(sm_count()) * 16;
  const int blocks = int(want < most ? want : most);
  if (a_dtype == PTB_F32)
    add_stream_kernel<float><<<blocks, threads, 0, stream>>>(x, (const float*)a, out, size_t(total));
  else if (a_dtype == PTB_BF16)
    add_stream_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>(x, (const __nv_bfloat16*)a, out, size_t(total));
  else
    return PTB_ERR_DTYPE;
  return launch_status();
}

// gain_next / next: null, or the next sublayer's norm of the new stream (out_dtype: its dtype)
PTB_API int ptb_post_norm_add(const float* x, int y_dtype, const void* y, const float* gain, float eps, float mult,
                              float* out, const float* gain_next, float eps_next, int next_dtype, void* next, int n,
                              int width, cudaStream_t stream) {
  if (n <= 0) return PTB_OK;
  if (width <= 0 || size_t(width) * 4 > 200 * 1024 || (gain_next == nullptr) != (next == nullptr)) return PTB_ERR_SIZE;
  const size_t smem = size_t(width) * sizeof(float);
  const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
#define PTB_PNA(TA, TO)                                                                                              \
  {                                                                                                                  \
    static size_t configured = 48 * 1024;                                                                            \
    if (smem > configured) {                                                                                         \
      if (cudaFuncSetAttribute(post_norm_add_kernel<TA, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize,            \
                               int(smem)) != cudaSuccess)                                                            \
        return PTB_ERR_LAUNCH;                                                                                       \
      configured = smem;                                                                                             \
    }                                                                                                                \
    post_norm_add_kernel<TA, TO><<<n, threads, smem, stream>>>(x, (const TA*)y, gain, eps, mult, out, gain_next,     \
                                                               eps_next, (TO*)next, width);                          \
  }
  const bool next16 = next != nullptr && next_dtype == PTB_BF16;
  if (next != nullptr && next_dtype != PTB_BF16 && next_dtype != PTB_F32) return PTB_ERR_DTYPE;
  if (y_dtype == PTB_F32) {
    if (next16) PTB_PNA(float, __nv_bfloat16) else PTB_PNA(float, float)
  } else if (y_dtype == PTB_BF16) {
    if (next16) PTB_PNA(__nv_bfloat16, __nv_bfloat16) else PTB_PNA(__nv_bfloat16, float)
  } else {
    return PTB_ERR_DTYPE;
  }
#undef PTB_PNA
  return launch_status();
}

PTB_API int ptb_embed_sum(int dtype, const int* ids, const int* pos, const void* table, const void* positions, float* out,
                          int n, int width, int rows, int pos_rows, int* status, cudaStream_t stream) {
  if (n <= 0) return PTB_OK;
  if (width <= 0 || rows <= 0 || pos_rows <= 0) return PTB_ERR_SIZE;
  const int threads = width >= 1024 ? 256 : 128;
  if (dtype == PTB_F32)
    embed_sum_kernel<float><<<n, threads, 0, stream>>>(ids, pos, (const float*)table, (const float*)positions, out, width,
                                                       rows, pos_rows, status);
  else if (dtype == PTB_BF16)
    embed_sum_kernel<__nv_bfloat16><<<n, threads, 0, stream>>>(ids, pos, (const __nv_bfloat16*)table,
                                                               (const __nv_bfloat16*)positions, out, width, rows,
                                                               pos_rows, status);
  else
    return PTB_ERR_DTYPE;
  return launch_status();
}
