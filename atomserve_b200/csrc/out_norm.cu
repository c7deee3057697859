// Kernels for blocks whose norm sits on the sublayer's output, x <- x + mult * norm(f(x)), over a
// float32 residual stream, and for the mixers such blocks carry. Everything inside is float32;
// each stored value is rounded once.
//
//   asb_residual_out_norm    out = x + mult * N(y) * gain * scale, N the centred norm
//                            (y - mean) / sqrt(var + eps) or the RMS norm y / sqrt(mean(y^2) + eps);
//                            scale (a per-channel layer scale) and x may be absent (x absent: the
//                            norm alone, with an optional row gather, as before an output head);
//                            y may be given as two halves, y = (R(a) ga + R(b) gb) / 2 with R the
//                            unit-RMS norm: two mixers that run side by side. Written as float32
//                            (the stream) and/or in the compute dtype (what the next products read).
//   asb_head_norm_gate       per head of `width` columns: o / sqrt(mean(o^2) + eps) (width 0: no
//                            norm), times gain (optional), times sigmoid or SiLU of a gate read
//                            from a projection's columns; before the norm, optionally divided by
//                            max(|nq|, exp(-top)) + floor per (token, head): a matrix memory's
//                            normaliser.
//   asb_projection_norm_store  queries and keys RMS-normed over their whole projection (all heads at
//                            once), the keys written to their pages, and the keys as projected
//                            written as the values.
//   asb_capped_gates_scan    a gated matrix memory's log gates i = cap tanh(zi / cap),
//                            f = logsigmoid(cap tanh(zf / cap)), the running maximum
//                            top_t = max(f_t + top_(t-1), i_t) per (request, head) carried in the
//                            request's state, and from them each token's decay
//                            exp(f_t + top_(t-1) - top_t) and input weight exp(i_t - top_t).
//   asb_gated_token_slice    act(z) * table[token, offset : offset + dim]: the gate of a per-layer
//                            token input.
#include "common.cuh"
#include "gemm_partials.cuh"

namespace {

__device__ __forceinline__ float gelu_tanh_f(float z) {
  return 0.5f * z * (1.f + tanhf(0.79788456080286536f * (z + 0.044715f * z * z * z)));
}

// One block per output row; the row is kept in shared memory between the passes.
template <typename T>
__global__ void residual_out_norm_kernel(float* __restrict__ out32, T* __restrict__ out_c, const float* __restrict__ x,
                                         const float* __restrict__ y, const float* __restrict__ y2,
                                         const float* __restrict__ gain_a, const float* __restrict__ gain_b,
                                         const float* __restrict__ gain, const float* __restrict__ scale,
                                         const int* __restrict__ rows, int width, float mult, float eps, int centred) {
  extern __shared__ float row[];
  __shared__ float scratch[32];
  asb::pdl_wait();
  asb::pdl_launch_dependents();
  const size_t src = rows ? (size_t)rows[blockIdx.x] : (size_t)blockIdx.x;
  const float* yr = y + src * width;
  const float inv_w = 1.f / (float)width;
  if (y2) {
    const float* br = y2 + src * width;
    float sa = 0.f, sb = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
      sa = fmaf(yr[i], yr[i], sa);
      sb = fmaf(br[i], br[i], sb);
    }
    const float ia = 1.f / sqrtf(asb::block_sum(sa, scratch) * inv_w + eps);
    const float ib = 1.f / sqrtf(asb::block_sum(sb, scratch) * inv_w + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x)
      row[i] = 0.5f * (yr[i] * ia * gain_a[i] + br[i] * ib * gain_b[i]);
  } else {
    for (int i = threadIdx.x; i < width; i += blockDim.x) row[i] = yr[i];
  }
  // (each thread reads back only what it wrote itself: no barrier is needed for `row`)
  float mean = 0.f;
  if (centred) {
    float s = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) s += row[i];
    mean = asb::block_sum(s, scratch) * inv_w;
  }
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float d = row[i] - mean;
    ss = fmaf(d, d, ss);
  }
  const float inv = 1.f / sqrtf(asb::block_sum(ss, scratch) * inv_w + eps);
  const float* xr = x ? x + src * width : nullptr;
  const size_t dst = (size_t)blockIdx.x * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float v = (row[i] - mean) * inv * gain[i];
    if (scale) v *= scale[i];
    v = xr ? fmaf(mult, v, xr[i]) : mult * v;
    if (out32) out32[dst + i] = v;
    if (out_c) out_c[dst + i] = asb::from_float<T>(v);
  }
}

// asb_residual_out_norm with y given as the partial sums that the tensor-core GEMM left in its
// workspace (few tokens): a thread adds up the slots of 8 columns itself, in the reduction's order,
// so the GEMM's reduction kernel and a round trip of y through memory fall away.
__global__ void partial_residual_out_norm_kernel(float* __restrict__ out32, __nv_bfloat16* __restrict__ out_c,
                                                 const asb::PartialSums ps, const float* __restrict__ x,
                                                 const float* __restrict__ gain, const float* __restrict__ scale,
                                                 int width, float mult, float eps, int centred) {
  __shared__ float scratch[32];
  const int t = blockIdx.x, i = threadIdx.x * 8;
  const bool active = i < width;
  const int slots = active ? asb::partial_slots(ps, i / asb::kPartialRows) : 0;
  asb::pdl_wait();
  asb::pdl_launch_dependents();
  float y[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) y[k] = 0.f;
  if (active) asb::partial_sum<8>(ps, t, i, slots, y);
  const float inv_w = 1.f / (float)width;
  float mean = 0.f;
  if (centred) {
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) s += y[k];
    mean = asb::block_sum(s, scratch) * inv_w;
  }
  float ss = 0.f;
  if (active) {
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float d = y[k] - mean;
      ss = fmaf(d, d, ss);
    }
  }
  const float inv = 1.f / sqrtf(asb::block_sum(ss, scratch) * inv_w + eps);
  if (!active) return;
  const float4 g0 = *reinterpret_cast<const float4*>(gain + i), g1 = *reinterpret_cast<const float4*>(gain + i + 4);
  const float4 x0 = *reinterpret_cast<const float4*>(x + (size_t)t * width + i);
  const float4 x1 = *reinterpret_cast<const float4*>(x + (size_t)t * width + i + 4);
  const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
  const float xs[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
  float v[8];
  uint4 packed;
  __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(&packed);
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    float n = (y[k] - mean) * inv * g[k];
    if (scale) n *= scale[i + k];
    v[k] = fmaf(mult, n, xs[k]);
    o[k] = __float2bfloat16_rn(v[k]);
  }
  *reinterpret_cast<float4*>(out32 + (size_t)t * width + i) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(out32 + (size_t)t * width + i + 4) = make_float4(v[4], v[5], v[6], v[7]);
  *reinterpret_cast<uint4*>(out_c + (size_t)t * width + i) = packed;
}

// One block per token, a warp per head (in turn). TO: the type of o.
template <typename T, typename TO>
__global__ void head_norm_gate_kernel(T* __restrict__ out, const TO* __restrict__ o, const T* __restrict__ gate,
                                      int gate_stride, const float* __restrict__ gain, const float* __restrict__ nq,
                                      const float* __restrict__ top, int heads, int width, int normed, float eps,
                                      float floor_, int silu) {
  asb::pdl_wait();
  asb::pdl_launch_dependents();
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  for (int h = warp; h < heads; h += nwarps) {
    const TO* oh = o + ((size_t)t * heads + h) * width;
    float div = 1.f;
    if (nq) div = 1.f / (fmaxf(fabsf(nq[(size_t)t * heads + h]), expf(-top[(size_t)t * heads + h])) + floor_);
    float inv = 1.f;
    if (normed) {
      float ss = 0.f;
      for (int i = lane; i < width; i += 32) {
        const float v = asb::to_float(oh[i]) * div;
        ss = fmaf(v, v, ss);
      }
      inv = 1.f / sqrtf(asb::warp_sum(ss) / (float)width + eps);
    }
    const T* g = gate + (size_t)t * gate_stride + h * width;
    for (int i = lane; i < width; i += 32) {
      float v = asb::to_float(oh[i]) * div * inv;
      if (gain) v *= gain[h * width + i];
      const float z = asb::to_float(g[i]);
      const float sg = 1.f / (1.f + expf(-z));
      out[((size_t)t * heads + h) * width + i] = asb::from_float<T>(v * (silu ? z * sg : sg));
    }
  }
}

// One block per token. proj row: queries at q_off (H * hd columns), keys at k_off (KV * hd columns).
template <typename T>
__global__ void projection_norm_store_kernel(T* __restrict__ q_out, const T* __restrict__ proj, int stride, int q_off,
                                             int k_off, const float* __restrict__ q_gain, const float* __restrict__ k_gain,
                                             const int* __restrict__ slots, T* __restrict__ k_cache, T* __restrict__ v_cache,
                                             int q_width, int KV, int hd, int bs, float eps) {
  __shared__ float scratch[32];
  asb::pdl_wait();
  asb::pdl_launch_dependents();
  const int t = blockIdx.x;
  const T* qr = proj + (size_t)t * stride + q_off;
  const T* kr = proj + (size_t)t * stride + k_off;
  const int k_width = KV * hd;
  float sq = 0.f, sk = 0.f;
  for (int i = threadIdx.x; i < q_width; i += blockDim.x) {
    const float v = asb::to_float(qr[i]);
    sq = fmaf(v, v, sq);
  }
  for (int i = threadIdx.x; i < k_width; i += blockDim.x) {
    const float v = asb::to_float(kr[i]);
    sk = fmaf(v, v, sk);
  }
  const float iq = 1.f / sqrtf(asb::block_sum(sq, scratch) / (float)q_width + eps);
  const float ik = 1.f / sqrtf(asb::block_sum(sk, scratch) / (float)k_width + eps);
  for (int i = threadIdx.x; i < q_width; i += blockDim.x)
    q_out[(size_t)t * q_width + i] = asb::from_float<T>(asb::to_float(qr[i]) * iq * q_gain[i]);
  const int slot = slots ? slots[t] : -1;
  if (slot < 0) return;  // a padding token: nothing is kept of it
  const size_t page = slot / bs, off = slot % bs;
  for (int i = threadIdx.x; i < k_width; i += blockDim.x) {
    const int g = i / hd, e = i - g * hd;
    const size_t at = ((page * KV + g) * bs + off) * hd + e;
    k_cache[at] = asb::from_float<T>(asb::to_float(kr[i]) * ik * k_gain[i]);
    v_cache[at] = kr[i];
  }
}

// One block per request, a warp per head (in turn), 32 tokens at a time: a lane turns its token's
// pre-activations into log gates; the running maximum is a scan of the maps x -> max(x + f, i),
// which compose as (f1, i1) then (f2, i2) = (f1 + f2, max(i1 + f2, i2)): five shuffle steps give
// every lane the map of the group's tokens up to its own, applied to the maximum the group
// starts from. Within a group the sums of f are grouped differently from token-by-token steps:
// equal beyond rounding.
__global__ void capped_gates_scan_kernel(float* __restrict__ decay, float* __restrict__ gain, float* __restrict__ top_out,
                                         const float* __restrict__ z, int z_stride, int i_off, int f_off,
                                         const float* __restrict__ i_bias, const float* __restrict__ f_bias,
                                         float* __restrict__ top_state, const int* __restrict__ state_slots,
                                         const int* __restrict__ req_q_start, int H, float cap) {
  asb::pdl_wait();
  asb::pdl_launch_dependents();
  const int r = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int lo = req_q_start[r], hi = req_q_start[r + 1];
  const float inv_cap = 1.f / cap;
  for (int h = warp; h < H; h += nwarps) {
    float* ts = top_state + (size_t)state_slots[r] * H + h;
    float top = *ts;  // the maximum before the group's first token (the same in every lane)
    const float bi = i_bias[h], bf = f_bias[h];
    for (int t0 = lo; t0 < hi; t0 += 32) {
      const int t = t0 + lane;
      const bool real = t < hi;
      float f = 0.f, i = -INFINITY;  // the identity map for lanes past the end
      if (real) {
        const float u = cap * tanhf((z[(size_t)t * z_stride + f_off + h] + bf) * inv_cap);
        f = fminf(u, 0.f) - log1pf(expf(-fabsf(u)));  // log sigmoid(u)
        i = cap * tanhf((z[(size_t)t * z_stride + i_off + h] + bi) * inv_cap);
      }
      float F = f, I = i;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const float pF = __shfl_up_sync(0xffffffffu, F, off), pI = __shfl_up_sync(0xffffffffu, I, off);
        if (lane >= off) {
          I = fmaxf(pI + F, I);
          F = pF + F;
        }
      }
      const float mine = fmaxf(top + F, I);
      float before = __shfl_up_sync(0xffffffffu, mine, 1);
      if (lane == 0) before = top;
      if (real) {
        const size_t at = (size_t)t * H + h;
        decay[at] = expf(f + before - mine);
        gain[at] = expf(i - mine);
        top_out[at] = mine;
      }
      top = __shfl_sync(0xffffffffu, mine, 31);  // (lanes past the end carry the last real maximum)
    }
    if (lane == 0) *ts = top;
  }
}

template <typename T>
__global__ void gated_token_slice_kernel(T* __restrict__ out, const float* __restrict__ z, const T* __restrict__ table,
                                         const int* __restrict__ ids, int table_width, int offset, int dim, int vocab,
                                         long long total) {
  asb::pdl_wait();
  asb::pdl_launch_dependents();
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / dim;
    const int j = (int)(idx - t * dim);
    const int id = ids[t];
    const float e = (id >= 0 && id < vocab) ? asb::to_float(table[(size_t)id * table_width + offset + j]) : 0.f;
    out[idx] = asb::from_float<T>(gelu_tanh_f(z[idx]) * e);
  }
}

int threads_for(int width) { return width >= 4096 ? 512 : (width >= 1024 ? 256 : 128); }

}  // namespace

// out32 and out_c: either may be null; dtype is that of out_c. x, scale, rows: may be null. y2 with
// gain_a and gain_b: all three or none.
extern "C" int asb_residual_out_norm(float* out32, void* out_c, const float* x, const float* y, const float* y2,
                                     const float* gain_a, const float* gain_b, const float* gain, const float* scale,
                                     const int* rows, int n, int width, float mult, float eps, int centred, int dtype,
                                     cudaStream_t stream) {
  if (n == 0) return 0;
  if (width < 1 || width > 12288) return asb::fail("residual_out_norm: width %d not in 1..12288", width);
  if (!y || !gain) return asb::fail("residual_out_norm: y and gain are required");
  if ((y2 != nullptr) != (gain_a != nullptr) || (y2 != nullptr) != (gain_b != nullptr))
    return asb::fail("residual_out_norm: two halves come with a gain each");
  const size_t smem = sizeof(float) * (size_t)width;
  ASB_DISPATCH_DTYPE(dtype, T, {
    auto kern = residual_out_norm_kernel<T>;
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return asb::fail("residual_out_norm: shared memory %zu: %s", smem, cudaGetErrorString(e));
    }
    asb::launch(kern, n, threads_for(width), smem, stream, out32, (T*)out_c, x, y, y2, gain_a, gain_b, gain, scale, rows,
                width, mult, eps, centred);
  });
  return asb::check_launch("residual_out_norm");
}

// out32 (float32) and out_c (bfloat16) = x + mult * N(y) * gain * scale, y being the partial sums of
// asb_gemm_tcgen05 mode 3 on [tokens, K] x [width, K]. Widths that are a multiple of 8 up to 8192,
// pointers 16-byte aligned. scale may be null.
extern "C" int asb_partial_residual_out_norm(float* out32, void* out_c, const float* ws, int max_slots, int bn,
                                             int kb_per_tile, int num_tiles, int blocks, const float* x,
                                             const float* gain, const float* scale, int tokens, int width, float mult,
                                             float eps, int centred, cudaStream_t stream) {
  if (tokens == 0) return 0;
  if (width % 8 || width / 8 > 1024) return asb::fail("partial_residual_out_norm: width %d must be a multiple of 8 up to 8192", width);
  if (tokens > bn || num_tiles * asb::kPartialRows < width)
    return asb::fail("partial_residual_out_norm: %d tokens x %d columns do not fit the partial sums (%d x %d)", tokens, width, bn,
                     num_tiles * asb::kPartialRows);
  if (((uintptr_t)out32 | (uintptr_t)out_c | (uintptr_t)x | (uintptr_t)gain | (uintptr_t)ws) & 15)
    return asb::fail("partial_residual_out_norm: pointers must be 16-byte aligned");
  const asb::PartialSums ps = {ws, max_slots, bn, kb_per_tile, num_tiles, blocks};
  const int threads = ((width / 8) + 31) / 32 * 32;
  asb::launch(partial_residual_out_norm_kernel, tokens, threads, 0, stream, out32, (__nv_bfloat16*)out_c, ps, x, gain, scale,
              width, mult, eps, centred);
  return asb::check_launch("partial_residual_out_norm");
}

// o: [n, heads * width], float32 (o_dtype 0) or the compute dtype (1: as `dtype`). gate: rows of
// gate_stride elements in the compute dtype. gain [heads * width], nq and top [n, heads]: optional.
extern "C" int asb_head_norm_gate(void* out, const void* o, int o_dtype, const void* gate, int gate_stride,
                                  const float* gain, const float* nq, const float* top, int n, int heads, int width,
                                  int normed, float eps, float floor_, int silu, int dtype, cudaStream_t stream) {
  if (n == 0) return 0;
  if (heads < 1 || width < 1) return asb::fail("head_norm_gate: %d heads of %d", heads, width);
  if ((nq != nullptr) != (top != nullptr)) return asb::fail("head_norm_gate: a normaliser comes with its running maximum");
  const int threads = heads >= 8 ? 256 : (heads >= 4 ? 128 : 32 * heads);
  ASB_DISPATCH_DTYPE(dtype, T, {
    if (o_dtype == asb::kFloat32)
      asb::launch(head_norm_gate_kernel<T, float>, n, threads, 0, stream, (T*)out, (const float*)o, (const T*)gate,
                  gate_stride, gain, nq, top, heads, width, normed, eps, floor_, silu);
    else
      asb::launch(head_norm_gate_kernel<T, T>, n, threads, 0, stream, (T*)out, (const T*)o, (const T*)gate, gate_stride,
                  gain, nq, top, heads, width, normed, eps, floor_, silu);
  });
  return asb::check_launch("head_norm_gate");
}

extern "C" int asb_projection_norm_store(void* q_out, const void* proj, int stride, int q_off, int k_off,
                                         const float* q_gain, const float* k_gain, const int* slots, void* k_cache,
                                         void* v_cache, int n, int H, int KV, int hd, int bs, float eps, int dtype,
                                         cudaStream_t stream) {
  if (n == 0) return 0;
  if (H < 1 || KV < 1 || hd < 1 || bs < 1) return asb::fail("projection_norm_store: %d heads, %d kv heads of %d, pages of %d", H, KV, hd, bs);
  ASB_DISPATCH_DTYPE(dtype, T, asb::launch(projection_norm_store_kernel<T>, n, threads_for(H * hd), 0, stream, (T*)q_out,
                                           (const T*)proj, stride, q_off, k_off, q_gain, k_gain, slots, (T*)k_cache,
                                           (T*)v_cache, H * hd, KV, hd, bs, eps));
  return asb::check_launch("projection_norm_store");
}

// z: float32 [T, z_stride], the input gate's pre-activations at i_off and the forget gate's at
// f_off (H columns each). decay, gain, top_out: float32 [T, H]. top_state: [slots, H].
extern "C" int asb_capped_gates_scan(float* decay, float* gain, float* top_out, const float* z, int z_stride, int i_off,
                                     int f_off, const float* i_bias, const float* f_bias, float* top_state,
                                     const int* state_slots, const int* req_q_start, int R, int H, float cap,
                                     cudaStream_t stream) {
  if (R == 0) return 0;
  if (H < 1 || !(cap > 0.f)) return asb::fail("capped_gates_scan: %d heads, cap %f", H, cap);
  const int threads = 32 * (H < 16 ? H : 16);
  asb::launch(capped_gates_scan_kernel, R, threads, 0, stream, decay, gain, top_out, z, z_stride, i_off, f_off, i_bias,
              f_bias, top_state, state_slots, req_q_start, H, cap);
  return asb::check_launch("capped_gates_scan");
}

extern "C" int asb_gated_token_slice(void* out, const float* z, const void* table, const int* ids, int n,
                                     int table_width, int offset, int dim, int vocab, int dtype, cudaStream_t stream) {
  if (n == 0 || dim == 0) return 0;
  if (offset < 0 || offset + dim > table_width) return asb::fail("gated_token_slice: columns %d..%d of %d", offset, offset + dim, table_width);
  const long long total = (long long)n * dim;
  const long long blocks = (total + 255) / 256;
  ASB_DISPATCH_DTYPE(dtype, T, asb::launch(gated_token_slice_kernel<T>, (unsigned)(blocks < 148 * 16 ? blocks : 148 * 16), 256, 0,
                                           stream, (T*)out, z, (const T*)table, ids, table_width, offset, dim, vocab, total));
  return asb::check_launch("gated_token_slice");
}
