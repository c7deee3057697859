// The routed experts' products for bfloat16 on the tensor cores: the same grouped rows, tiles
// and results as the CUDA-core kernels of moe.cu (which stay the float32 path and the fallback),
// with mma.sync m16n8k16 (bfloat16 in, float32 accumulate). A block computes a 64 x 64 or a
// 128 x 64 tile of one expert's rows: warps of 32 x 32 each, K in steps of 32 brought to shared
// memory by 16-byte cp.async into two buffers (the next step arriving while this one is
// multiplied), fragments by ldmatrix. Each output
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

constexpr int BN = 64, BK = 32, LD = BK + 8;  // LD: row stride in shared memory, conflict-free for ldmatrix
constexpr int kStages = 2;

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

__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], const uint32_t* b) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* row) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(row);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

__device__ __forceinline__ void copy16(void* dst, const void* src, bool real) {
  // 16 bytes global -> shared without passing registers; `real` false writes zeros instead
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(real ? 16 : 0) : "memory");
}

// WM warps along the rows (2: tiles of 64 rows, 4 warps; 4: tiles of 128 rows, 8 warps), two along
// the columns; a warp computes 32 x 32 (and the same of the up matrix with GLU).
template <bool GLU, int WM>
__global__ void __launch_bounds__(WM * 64)
grouped_gemm_mma_kernel(const GroupedParams p) {
  constexpr int BM = WM * 32, kThreads = WM * 64;
  asb::pdl_wait();
  asb::pdl_launch_dependents();
  __shared__ __align__(16) __nv_bfloat16 xs[kStages][BM][LD];
  __shared__ __align__(16) __nv_bfloat16 ws[kStages][BN][LD];
  __shared__ __align__(16) __nv_bfloat16 us[GLU ? kStages : 1][GLU ? BN : 1][LD];
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

  // a stage: BM x 4 chunks of x, 64 x 4 of each weight tile, 16 bytes each, by cp.async
  auto request = [&](int k0, int stage) {
    for (int i = tid; i < BM * 4; i += kThreads) {
      const int r = i >> 2, k = k0 + (i & 3) * 8;
      const int xr = src_row[r];
      const bool real = xr >= 0 && k < K;
      copy16(&xs[stage][r][(i & 3) * 8], real ? p.x + (size_t)xr * K + k : p.x, real);
    }
    for (int i = tid; i < BN * 4; i += kThreads) {
      const int r = i >> 2, k = k0 + (i & 3) * 8;
      const bool real = n0 + r < N && k < K;
      copy16(&ws[stage][r][(i & 3) * 8], real ? w + (size_t)(n0 + r) * K + k : w, real);
      if constexpr (GLU) copy16(&us[stage][r][(i & 3) * 8], real ? w2 + (size_t)(n0 + r) * K + k : w2, real);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
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
  // ldmatrix rows. A: row lane % 16 of a 16-row tile, k block lane / 16. B: row (lane % 8) + 8 * (lane / 16)
  // of a pair of 8-column tiles, k block (lane / 8) % 2.
  const int a_row = wm + (lane & 15), a_col = (lane >> 4) * 8;
  const int b_row = wn + (lane & 7) + ((lane >> 4) & 1) * 8, b_col = ((lane >> 3) & 1) * 8;

  request(0, 0);
  for (int k0 = 0, stage = 0; k0 < K; k0 += BK, stage ^= 1) {
    if (k0 + BK < K) {
      request(k0 + BK, stage ^ 1);  // that buffer was read two steps ago, before the barrier that ended the last step
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; kk += 16) {
      uint32_t a[2][4];
      ldmatrix_x4(a[0], &xs[stage][a_row][kk + a_col]);
      ldmatrix_x4(a[1], &xs[stage][a_row + 16][kk + a_col]);
#pragma unroll
      for (int jp = 0; jp < 2; ++jp) {  // a pair of 8-column tiles per ldmatrix
        uint32_t b[4];
        ldmatrix_x4(b, &ws[stage][b_row + jp * 16][kk + b_col]);
        mma_bf16(acc[0][2 * jp], a[0], b);
        mma_bf16(acc[1][2 * jp], a[1], b);
        mma_bf16(acc[0][2 * jp + 1], a[0], b + 2);
        mma_bf16(acc[1][2 * jp + 1], a[1], b + 2);
        if constexpr (GLU) {
          ldmatrix_x4(b, &us[stage][b_row + jp * 16][kk + b_col]);
          mma_bf16(acc2[0][2 * jp], a[0], b);
          mma_bf16(acc2[1][2 * jp], a[1], b);
          mma_bf16(acc2[0][2 * jp + 1], a[0], b + 2);
          mma_bf16(acc2[1][2 * jp + 1], a[1], b + 2);
        }
      }
    }
    __syncthreads();  // this stage has been read: the step after next may overwrite it
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

// Tiles of 128 rows once the experts have 64 rows each on average; below that the tiles of 64
// rows waste less of the tensor cores' work on rows that do not exist.
bool tall(int pairs, int E) { return pairs >= 64 * E; }

int row_tiles(int pairs, int E, int bm) { return pairs / bm + (pairs < E ? pairs : E); }

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
  const bool big = tall(pairs, E);
  dim3 grid((F + BN - 1) / BN, row_tiles(pairs, E, big ? 128 : 64));
  if (grid.y > 65535) return asb::fail("moe_glu_mma: %d rows exceed the grid", pairs);
  if (big) asb::launch(grouped_gemm_mma_kernel<true, 4>, grid, 256, 0, stream, p);
  else asb::launch(grouped_gemm_mma_kernel<true, 2>, grid, 128, 0, stream, p);
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
  const bool big = tall(pairs, E);
  dim3 grid((N + BN - 1) / BN, row_tiles(pairs, E, big ? 128 : 64));
  if (grid.y > 65535) return asb::fail("moe_down_mma: %d rows exceed the grid", pairs);
  if (big) asb::launch(grouped_gemm_mma_kernel<false, 4>, grid, 256, 0, stream, p);
  else asb::launch(grouped_gemm_mma_kernel<false, 2>, grid, 128, 0, stream, p);
  return asb::check_launch("moe_down_mma");
}
