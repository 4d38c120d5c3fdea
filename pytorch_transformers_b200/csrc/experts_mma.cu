// The experts' grouped matrix products in bfloat16 on the tensor cores (mma.m16n8k16, float32 sums):
// the tiles of the plan that expert_plan_kernel makes (csrc/experts.cu), 64 or 128 sorted rows of one expert
// each. A block of 4 or 8 warps takes one tile x 128 rows of the expert's matrix; a warp owns 32 rows of the
// tile and 64 of the 128 matrix rows. Operands come through a three-stage cp.async ring of [rows][32] tiles whose
// 16-byte chunks are XOR-swizzled so that ldmatrix meets no bank twice.
//   mode 0: x rows are gathered from h by token; the 128 matrix rows are 64 gate rows and the 64 up rows
//           of the same columns; out[row, f] = silu(gate) * up, bfloat16.
//   mode 1: x rows are the sorted rows themselves; out[row, n] float32.
//   mode 2: x rows gathered as in mode 0, 128 plain matrix rows; out[row, n] = act(row_scale[pair] * sum), bfloat16
//           (an expert without a gate whose input is the token's row times the pair's weight).
// A row's sums do not depend on its place in a tile or on the other rows.
#include "mma_common.cuh"

namespace {

constexpr int GB = 128, GK = 32, STAGES = 3;   // matrix rows of a block, step along K, stages of the ring

// byte offset of 16-byte chunk c (0..3) of row r in a [rows][32] bfloat16 tile
__device__ __forceinline__ uint32_t gswz(int r, int c) { return uint32_t(r * 64 + ((c ^ ((r >> 1) & 3)) << 4)); }

// GM: rows of a tile (64: 4 warps, or 128: 8 warps, which halves the matrix's bytes per product where experts
// have that many rows); a warp owns 32 rows x 64 staged matrix rows.
template <int MODE, int GM>
__global__ void __launch_bounds__(2 * GM)
expert_linear_mma_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w, void* __restrict__ out_v,
                         const int* __restrict__ plan, int pairs, int max_tiles, int top, int N, int K,
                         const float* __restrict__ row_scale, int act) {
  const int tile = blockIdx.y;
  if (tile >= plan[0]) return;
  const int expert = plan[1 + tile], row0 = plan[1 + max_tiles + tile], rows = plan[1 + 2 * max_tiles + tile];
  const int* pair_of_row = plan + 1 + 3 * max_tiles + pairs;
  constexpr int GTHREADS = 2 * GM, B_COPIES = GB * 4 / GTHREADS;
  extern __shared__ __align__(128) unsigned char gsm[];
  unsigned char (*a_s)[GM * 64] = reinterpret_cast<unsigned char (*)[GM * 64]>(gsm);
  unsigned char (*b_s)[GB * 64] = reinterpret_cast<unsigned char (*)[GB * 64]>(gsm + STAGES * GM * 64);
  int* src_row = reinterpret_cast<int*>(gsm + STAGES * (GM + GB) * 64);
  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  constexpr int NOUT = MODE == 0 ? 64 : 128;     // output columns of a block
  const int n0 = blockIdx.x * NOUT;
  if (tid < GM) src_row[tid] = (tid < rows) ? (MODE != 1 ? pair_of_row[row0 + tid] / top : row0 + tid) : -1;
  __syncthreads();
  const __nv_bfloat16* we = w + size_t(expert) * (MODE == 0 ? 2 : 1) * N * K;

  // what this thread copies in every stage: 2 chunks of the rows' tile and 4 or 2 of the matrix's, at fixed
  // places; only k moves (addresses and bounds are worked out once, not in the loop)
  const __nv_bfloat16* a_src[2];
  uint32_t a_off[2];
  const __nv_bfloat16* b_src[B_COPIES];
  uint32_t b_off[B_COPIES];
  const int kc = (tid % 4) * 8;       // this thread's chunk of a row: k0 + kc .. + 7
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int r = (tid + j * GTHREADS) / 4;
    a_off[j] = gswz(r, tid % 4);
    const int sr = src_row[r];
    a_src[j] = sr >= 0 ? x + size_t(sr) * K + kc : nullptr;
  }
#pragma unroll
  for (int j = 0; j < B_COPIES; ++j) {
    const int r = (tid + j * GTHREADS) / 4;
    b_off[j] = gswz(r, tid % 4);
    // row of the expert's matrix. mode 0: staged rows 64 nh + 32 part + cc hold column n0 + 32 nh + cc of the gate
    // (part 0) or up (part 1) rows, so that a warp (one nh) has both for its 32 columns
    int gn, col;
    if (MODE == 0) {
      col = n0 + (r >> 6) * 32 + (r & 31);
      gn = ((r >> 5) & 1) ? N + col : col;
    } else {
      col = gn = n0 + r;
    }
    b_src[j] = col < N ? we + size_t(gn) * K + kc : nullptr;
  }
  auto load_stage = [&](int stage, int k0) {
    const bool k_ok = k0 + kc < K;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      if (a_src[j] != nullptr && k_ok) cp_async16(smem_u32(a_s[stage]) + a_off[j], a_src[j] + k0);
      else *reinterpret_cast<uint4*>(a_s[stage] + a_off[j]) = make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int j = 0; j < B_COPIES; ++j) {
      if (b_src[j] != nullptr && k_ok) cp_async16(smem_u32(b_s[stage]) + b_off[j], b_src[j] + k0);
      else *reinterpret_cast<uint4*>(b_s[stage] + b_off[j]) = make_uint4(0, 0, 0, 0);
    }
  };

  const int wm = warp >> 1, wn = warp & 1;     // this warp: rows 32 wm .. + 31, staged matrix rows 64 wn .. + 63
  float acc[2][8][4];
#pragma unroll
  for (int mi = 0; mi < 2; ++mi)
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int q = 0; q < 4; ++q) acc[mi][j][q] = 0.f;

  const int k_tiles = (K + GK - 1) / GK;
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < k_tiles) load_stage(s, s * GK);
    cp_async_commit();
  }
  for (int kt = 0; kt < k_tiles; ++kt) {
    cp_async_wait<STAGES - 2>();
    __syncthreads();   // stage kt has landed for everybody, and stage kt - 1 is no longer read
    const int nxt = kt + STAGES - 1;
    if (nxt < k_tiles) load_stage(nxt % STAGES, nxt * GK);
    cp_async_commit();
    const int st = kt % STAGES;
    const uint32_t a_base = smem_u32(a_s[st]), b_base = smem_u32(b_s[st]);
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
      uint32_t a[2][4];
#pragma unroll
      for (int mi = 0; mi < 2; ++mi)
        ldmatrix_x4(a[mi][0], a[mi][1], a[mi][2], a[mi][3],
                    a_base + gswz(wm * 32 + mi * 16 + (lane & 15), ks * 2 + (lane >> 4)));
#pragma unroll
      for (int jp = 0; jp < 4; ++jp) {     // two fragments of 8 columns at a time
        uint32_t b0, b1, b2, b3;
        const int id = lane >> 3;
        ldmatrix_x4(b0, b1, b2, b3, b_base + gswz(wn * 64 + jp * 16 + (id >> 1) * 8 + (lane & 7), ks * 2 + (id & 1)));
#pragma unroll
        for (int mi = 0; mi < 2; ++mi) {
          mma_bf16(acc[mi][2 * jp], a[mi], b0, b1);
          mma_bf16(acc[mi][2 * jp + 1], a[mi], b2, b3);
        }
      }
    }
  }
  cp_async_wait<0>();
  const int c0 = (lane % 4) * 2;
#pragma unroll
  for (int mi = 0; mi < 2; ++mi) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = wm * 32 + mi * 16 + half * 8 + lane / 4;
      if (r >= rows) continue;
      if (MODE == 0) {
        __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out_v) + size_t(row0 + r) * N;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            const int col = n0 + wn * 32 + j * 8 + c0 + q;
            if (col >= N) continue;
            const float g = acc[mi][j][half * 2 + q], u = acc[mi][j + 4][half * 2 + q];
            o[col] = __float2bfloat16_rn(g / (1.f + expf(-g)) * u);
          }
        }
      } else if (MODE == 2) {
        __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out_v) + size_t(row0 + r) * N;
        const float rs = row_scale ? row_scale[pair_of_row[row0 + r]] : 1.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            const int col = n0 + wn * 64 + j * 8 + c0 + q;
            if (col < N) o[col] = __float2bfloat16_rn(apply_activation(acc[mi][j][half * 2 + q] * rs, act));
          }
        }
      } else {
        float* o = reinterpret_cast<float*>(out_v) + size_t(row0 + r) * N;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            const int col = n0 + wn * 64 + j * 8 + c0 + q;
            if (col < N) o[col] = acc[mi][j][half * 2 + q];
          }
        }
      }
    }
  }
}

}  // namespace

// rows of a tile that this kernel takes (the plan must be made with it)
PTB_API int ptb_expert_linear_mma_tile_rows() { return 64; }

namespace {
template <int MODE, int GM>
int launch_expert_mma(const void* x, const void* w, void* out, const int* plan, int pairs, int max_tiles, int top, int N,
                      int K, const float* row_scale, int act, cudaStream_t stream) {
  const size_t smem = size_t(STAGES) * (GM + GB) * 64 + GM * sizeof(int);
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(expert_linear_mma_kernel<MODE, GM>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) !=
        cudaSuccess)
      return PTB_ERR_LAUNCH;
    configured = true;
  }
  dim3 grid((N + (MODE == 0 ? 63 : 127)) / (MODE == 0 ? 64 : 128), max_tiles);
  expert_linear_mma_kernel<MODE, GM><<<grid, 2 * GM, smem, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w, out,
                                                                      plan, pairs, max_tiles, top, N, K, row_scale, act);
  return launch_status();
}
}  // namespace

// `tile_rows`: 64 or 128, the rows of the plan's tiles
PTB_API int ptb_expert_linear_mma(int mode, const void* x, const void* w, void* out, const int* plan, int pairs,
                                  int max_tiles, int top, int N, int K, int tile_rows, const float* row_scale, int act,
                                  cudaStream_t stream) {
  if (pairs <= 0 || max_tiles <= 0) return PTB_OK;
  if (N <= 0 || K <= 0 || K % 8 != 0 || max_tiles > 65535 || top <= 0 || (tile_rows != 64 && tile_rows != 128) ||
      mode < 0 || mode > 2 || !activation_known(act))
    return PTB_ERR_SIZE;
  if (!aligned16(x) || !aligned16(w)) return PTB_ERR_ALIGN;
#define PTB_EM(MM, GG) launch_expert_mma<MM, GG>(x, w, out, plan, pairs, max_tiles, top, N, K, row_scale, act, stream)
  if (mode == 0) return tile_rows == 64 ? PTB_EM(0, 64) : PTB_EM(0, 128);
  if (mode == 2) return tile_rows == 64 ? PTB_EM(2, 64) : PTB_EM(2, 128);
  return tile_rows == 64 ? PTB_EM(1, 64) : PTB_EM(1, 128);
#undef PTB_EM
}
