// The routed experts' products for bfloat16 on the tensor cores: the same grouped rows, tiles
// and results as the CUDA-core kernels of moe.cu (which stay the float32 path and the fallback),
// with mma.sync m16n8k16 (bfloat16 in, float32 accumulate). A block computes a 64 x 64 tile of
// one expert's rows: four warps of 32 x 32 each, K in steps of 32 staged through shared memory,
// the next step's global loads in flight while the current one is multiplied. Each output
// element is one float32 accumulator chain over k in ascending order, so a row's result does not
// depend on which rows share its tile.
//
//   asb_moe_glu_mma    hidden[row] = act(x[token] . gate_e^T, x[token] . up_e^T)   (bfloat16)
//   asb_moe_down_mma   y[row] = hidden[row] . down_e^T                            (float32)
//
// K must be a multiple of 8 and the operands 16-byte aligned (16-byte loads); the callers send
// other shapes to the CUDA-core kernels.
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 32, LD = BK + 8;  // LD: row stride in shared memory, conflict-free for the fragment loads

struct GroupedParams {
  void* out;
  const __nv_bfloat16* x;
  const int* row_token;
  const int* offsets;
  const __nv_bfloat16* w;
  const __nv_bfloat16* w2;
  int E, N, K;
  float limit, slope, shift;
};

__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

template <bool GLU>
__global__ void __launch_bounds__(128)
grouped_gemm_mma_kernel(const GroupedParams p) {
  asb::pdl_wait();
  asb::pdl_launch_dependents();
  __shared__ __align__(16) __nv_bfloat16 xs[BM][LD];
  __shared__ __align__(16) __nv_bfloat16 ws[BN][LD];
  __shared__ __align__(16) __nv_bfloat16 us[GLU ? BN : 1][LD];
  __shared__ int src_row[BM];
  int tile = blockIdx.y, e = 0, begin = 0, count = 0;
  for (; e < p.E; ++e) {
    begin = p.offsets[e];
    count = p.offsets[e + 1] - begin;
    const int tiles = (count + BM - 1) / BM;
    if (tile < tiles) break;
    tile -= tiles;
  }
  if (e == p.E) return;
  const int m0 = tile * BM, n0 = blockIdx.x * BN;
  const int rows = min(BM, count - m0);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid < BM) src_row[tid] = tid < rows ? (GLU ? p.row_token[begin + m0 + tid] : begin + m0 + tid) : -1;
  __syncthreads();
  const int K = p.K, N = p.N;
  const __nv_bfloat16* w = p.w + (size_t)e * N * K;
  const __nv_bfloat16* w2 = GLU ? p.w2 + (size_t)e * N * K : nullptr;
  // loads: 64 rows x 4 chunks of 8 values per operand tile; a thread takes chunk tid and tid + 128
  const int lrow0 = tid >> 2, lrow1 = lrow0 + 32, lchunk = (tid & 3) * 8;
  const int xr0 = src_row[lrow0], xr1 = src_row[lrow1];
  const int wn0 = n0 + lrow0, wn1 = n0 + lrow1;
  uint4 rx[2], rw[2], ru[2];
  const uint4 zero = make_uint4(0, 0, 0, 0);
  auto fetch = [&](int k0) {
    const int k = k0 + lchunk;
    const bool in = k < K;
    rx[0] = (in && xr0 >= 0) ? *reinterpret_cast<const uint4*>(p.x + (size_t)xr0 * K + k) : zero;
    rx[1] = (in && xr1 >= 0) ? *reinterpret_cast<const uint4*>(p.x + (size_t)xr1 * K + k) : zero;
    rw[0] = (in && wn0 < N) ? *reinterpret_cast<const uint4*>(w + (size_t)wn0 * K + k) : zero;
    rw[1] = (in && wn1 < N) ? *reinterpret_cast<const uint4*>(w + (size_t)wn1 * K + k) : zero;
    if constexpr (GLU) {
      ru[0] = (in && wn0 < N) ? *reinterpret_cast<const uint4*>(w2 + (size_t)wn0 * K + k) : zero;
      ru[1] = (in && wn1 < N) ? *reinterpret_cast<const uint4*>(w2 + (size_t)wn1 * K + k) : zero;
    }
  };
  auto stage = [&]() {
    *reinterpret_cast<uint4*>(&xs[lrow0][lchunk]) = rx[0];
    *reinterpret_cast<uint4*>(&xs[lrow1][lchunk]) = rx[1];
    *reinterpret_cast<uint4*>(&ws[lrow0][lchunk]) = rw[0];
    *reinterpret_cast<uint4*>(&ws[lrow1][lchunk]) = rw[1];
    if constexpr (GLU) {
      *reinterpret_cast<uint4*>(&us[lrow0][lchunk]) = ru[0];
      *reinterpret_cast<uint4*>(&us[lrow1][lchunk]) = ru[1];
    }
  };
  const int wm = (warp >> 1) * 32, wn = (warp & 1) * 32;  // the warp's 32 x 32 corner of the tile
  const int g = lane >> 2, t = lane & 3;
  float acc[2][4][4], acc2[GLU ? 2 : 1][4][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        acc[i][j][c] = 0.f;
        if constexpr (GLU) acc2[i][j][c] = 0.f;
      }
  fetch(0);
  for (int k0 = 0; k0 < K; k0 += BK) {
    __syncthreads();  // the previous step's fragments have been read
    stage();
    __syncthreads();
    if (k0 + BK < K) fetch(k0 + BK);
#pragma unroll
    for (int kk = 0; kk < BK; kk += 16) {
      uint32_t a[2][4];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int r = wm + i * 16 + g;
        a[i][0] = *reinterpret_cast<const uint32_t*>(&xs[r][kk + 2 * t]);
        a[i][1] = *reinterpret_cast<const uint32_t*>(&xs[r + 8][kk + 2 * t]);
        a[i][2] = *reinterpret_cast<const uint32_t*>(&xs[r][kk + 2 * t + 8]);
        a[i][3] = *reinterpret_cast<const uint32_t*>(&xs[r + 8][kk + 2 * t + 8]);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int n = wn + j * 8 + g;
        uint32_t b[2];
        b[0] = *reinterpret_cast<const uint32_t*>(&ws[n][kk + 2 * t]);
        b[1] = *reinterpret_cast<const uint32_t*>(&ws[n][kk + 2 * t + 8]);
        mma_bf16(acc[0][j], a[0], b);
        mma_bf16(acc[1][j], a[1], b);
        if constexpr (GLU) {
          b[0] = *reinterpret_cast<const uint32_t*>(&us[n][kk + 2 * t]);
          b[1] = *reinterpret_cast<const uint32_t*>(&us[n][kk + 2 * t + 8]);
          mma_bf16(acc2[0][j], a[0], b);
          mma_bf16(acc2[1][j], a[1], b);
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int m = wm + i * 16 + g + half * 8;
      if (m >= rows) continue;
      const size_t orow = (size_t)(begin + m0 + m) * N;
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int n = n0 + wn + j * 8 + 2 * t + c;
          if (n >= N) continue;
          float v = acc[i][j][half * 2 + c];
          if constexpr (GLU) {
            float gate = v, up = acc2[i][j][half * 2 + c];
            if (p.limit > 0.f) {
              gate = fminf(gate, p.limit);
              up = fminf(fmaxf(up, -p.limit), p.limit);
            }
            ((__nv_bfloat16*)p.out)[orow + n] = __float2bfloat16_rn(gate / (1.f + expf(-p.slope * gate)) * (up + p.shift));
          } else {
            ((float*)p.out)[orow + n] = v;
          }
        }
    }
}

int row_tiles(int pairs, int E) { return pairs / BM + (pairs < E ? pairs : E); }

bool aligned16(const void* a, const void* b, const void* c) {
  return (((uintptr_t)a | (uintptr_t)b | (uintptr_t)c) & 15) == 0;
}

}  // namespace

extern "C" int asb_moe_mma_supported(int K) { return K >= 8 && K % 8 == 0; }

extern "C" int asb_moe_glu_mma(void* hidden, const void* x, const int* row_token, const int* offsets, const void* gate,
                               const void* up, int pairs, int E, int F, int K, float limit, float slope, float shift,
                               cudaStream_t stream) {
  if (pairs == 0) return 0;
  if (!asb_moe_mma_supported(K) || !aligned16(x, gate, up)) return asb::fail("moe_glu_mma: K = %d must be a multiple of 8 and the operands 16-byte aligned", K);
  GroupedParams p;
  p.out = hidden; p.x = (const __nv_bfloat16*)x; p.row_token = row_token; p.offsets = offsets;
  p.w = (const __nv_bfloat16*)gate; p.w2 = (const __nv_bfloat16*)up;
  p.E = E; p.N = F; p.K = K; p.limit = limit; p.slope = slope; p.shift = shift;
  dim3 grid((F + BN - 1) / BN, row_tiles(pairs, E));
  if (grid.y > 65535) return asb::fail("moe_glu_mma: %d rows exceed the grid", pairs);
  asb::launch(grouped_gemm_mma_kernel<true>, grid, 128, 0, stream, p);
  return asb::check_launch("moe_glu_mma");
}

extern "C" int asb_moe_down_mma(float* y, const void* hidden, const int* offsets, const void* down, int pairs, int E,
                                int N, int F, cudaStream_t stream) {
  if (pairs == 0) return 0;
  if (!asb_moe_mma_supported(F) || !aligned16(hidden, down, nullptr)) return asb::fail("moe_down_mma: K = %d must be a multiple of 8 and the operands 16-byte aligned", F);
  GroupedParams p;
  p.out = y; p.x = (const __nv_bfloat16*)hidden; p.row_token = nullptr; p.offsets = offsets;
  p.w = (const __nv_bfloat16*)down; p.w2 = nullptr;
  p.E = E; p.N = N; p.K = F; p.limit = 0.f; p.slope = 1.f; p.shift = 0.f;
  dim3 grid((N + BN - 1) / BN, row_tiles(pairs, E));
  if (grid.y > 65535) return asb::fail("moe_down_mma: %d rows exceed the grid", pairs);
  asb::launch(grouped_gemm_mma_kernel<false>, grid, 128, 0, stream, p);
  return asb::check_launch("moe_down_mma");
}
