// Linear attention with a fixed decay per head ("lightning attention"), as a recurrence over a
// request's tokens:
//
//   S_t = decay_h S_(t-1) + k_t v_t^T        S: [D, V] per (request, head), float32, kept in the
//   o_t = S_t^T q_t                          request's state slot between steps
//
// q, k and v are column ranges of one projection [T, stride] in the compute dtype; `act` 1
// applies SiLU to them on the way in (float32). The state, the outer products, the decay and
// the outputs are float32.
//
// Work split: grid (request, head, chunk of value columns). A thread owns one value column and
// RPT rows of S in registers (D is covered by DS = 2^n adjacent lanes of RPT rows each, whose
// partial outputs are added by shuffles), so a token costs no block-wide synchronisation: a
// tile of TT tokens is staged in shared memory at once and walked in registers. The tokens of a
// request are walked in order whatever the step holds (a whole prompt, a portion, one decoded
// token), so the result does not depend on how a prompt was cut.
#include "common.cuh"

namespace {

constexpr int kThreads = 128;
constexpr int kTokenTile = 16;

struct LightningParams {
  float* out;               // [T, H * V]
  const void* proj;         // [T, stride]
  float* state;             // [slots, H, D, V]
  const int* state_slots;   // [R]
  const int* req_q_start;   // [R + 1]
  const float* decay;       // [H]
  int stride, q_off, k_off, v_off;
  int H, D, V, DS, act;
};

__device__ __forceinline__ float silu(float z) { return z / (1.f + expf(-z)); }

template <typename T, int RPT>
__global__ void __launch_bounds__(kThreads)
lightning_kernel(const LightningParams p) {
  asb::pdl_wait();
  asb::pdl_launch_dependents();
  extern __shared__ float smem[];
  const int DS = p.DS, DP = DS * RPT;    // padded rows
  const int CPB = kThreads / DS;          // value columns per block
  float* qs = smem;                       // [TT][DP]
  float* ks = qs + kTokenTile * DP;       // [TT][DP]
  float* vs = ks + kTokenTile * DP;       // [TT][CPB]
  const int r = blockIdx.x, h = blockIdx.y;
  const int ds = threadIdx.x % DS, cl = threadIdx.x / DS;
  const int col = blockIdx.z * CPB + cl;
  const int row_lo = p.req_q_start[r], row_hi = p.req_q_start[r + 1];
  const int slot = p.state_slots[r];
  const float dec = p.decay[h];
  const bool live = col < p.V;
  float* sp = p.state + (((size_t)slot * p.H + h) * p.D) * p.V + col;

  float S[RPT];
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int d = ds * RPT + i;
    S[i] = (live && d < p.D) ? sp[(size_t)d * p.V] : 0.f;
  }
  const T* proj = (const T*)p.proj;
  for (int t0 = row_lo; t0 < row_hi; t0 += kTokenTile) {
    const int nt = min(kTokenTile, row_hi - t0);
    __syncthreads();
    for (int i = threadIdx.x; i < nt * DP; i += kThreads) {
      const int t = i / DP, d = i - t * DP;
      float qv = 0.f, kv = 0.f;
      if (d < p.D) {
        const T* row = proj + (size_t)(t0 + t) * p.stride + h * p.D + d;
        qv = asb::to_float(row[p.q_off]);
        kv = asb::to_float(row[p.k_off]);
        if (p.act) { qv = silu(qv); kv = silu(kv); }
      }
      qs[i] = qv;
      ks[i] = kv;
    }
    for (int i = threadIdx.x; i < nt * CPB; i += kThreads) {
      const int t = i / CPB, c = blockIdx.z * CPB + (i - t * CPB);
      float vv = 0.f;
      if (c < p.V) {
        vv = asb::to_float(proj[(size_t)(t0 + t) * p.stride + p.v_off + h * p.V + c]);
        if (p.act) vv = silu(vv);
      }
      vs[i] = vv;
    }
    __syncthreads();
    for (int t = 0; t < nt; ++t) {
      const float vv = vs[t * CPB + cl];
      const float* kr = ks + t * DP + ds * RPT;
      const float* qr = qs + t * DP + ds * RPT;
      float o = 0.f;
#pragma unroll
      for (int i = 0; i < RPT; ++i) {
        S[i] = fmaf(dec, S[i], kr[i] * vv);
        o = fmaf(S[i], qr[i], o);
      }
      for (int off = 1; off < DS; off <<= 1) o += __shfl_xor_sync(0xffffffffu, o, off);
      if (ds == 0 && live) p.out[(size_t)(t0 + t) * p.H * p.V + h * p.V + col] = o;
    }
  }
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int d = ds * RPT + i;
    if (live && d < p.D) sp[(size_t)d * p.V] = S[i];
  }
}

template <typename T, int RPT>
int launch(const LightningParams& p, int R, cudaStream_t stream) {
  const int CPB = kThreads / p.DS;
  const size_t smem = sizeof(float) * kTokenTile * (2 * p.DS * RPT + CPB);
  auto kern = lightning_kernel<T, RPT>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return asb::fail("lightning_attention: shared memory %zu: %s", smem, cudaGetErrorString(e));
  dim3 grid(R, p.H, (p.V + CPB - 1) / CPB);
  asb::launch(kern, grid, kThreads, smem, stream, p);
  return asb::check_launch("lightning_attention");
}

}  // namespace

extern "C" int asb_lightning_attention(float* out, const void* proj, int stride, int q_off, int k_off, int v_off,
                                       float* state, const int* state_slots, const int* req_q_start,
                                       const float* decay, int R, int H, int D, int V, int act, int dtype,
                                       cudaStream_t stream) {
  if (R == 0) return 0;
  if (H < 1 || D < 1 || V < 1 || H > 65535) return asb::fail("lightning_attention: %d heads of %d x %d", H, D, V);
  LightningParams p;
  p.out = out; p.proj = proj; p.state = state; p.state_slots = state_slots; p.req_q_start = req_q_start;
  p.decay = decay; p.stride = stride; p.q_off = q_off; p.k_off = k_off; p.v_off = v_off;
  p.H = H; p.D = D; p.V = V; p.act = act;
  // rows of the state per thread: 64 from D = 64 on, fewer for narrow heads; D beyond 64 is
  // shared among 2, 4, ... lanes
  const int rpt = D >= 64 ? 64 : (D > 16 ? 32 : 16);
  int ds = 1;
  while (ds * rpt < D) ds <<= 1;
  if (ds > 32) return asb::fail("lightning_attention: key size %d exceeds %d", D, 32 * 64);
  p.DS = ds;
  if ((V + kThreads / ds - 1) / (kThreads / ds) > 65535) return asb::fail("lightning_attention: value size %d", V);
  ASB_DISPATCH_DTYPE(dtype, T, {
    if (rpt == 64) return launch<T, 64>(p, R, stream);
    if (rpt == 32) return launch<T, 32>(p, R, stream);
    return launch<T, 16>(p, R, stream);
  });
  return 0;
}
