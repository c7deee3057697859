// Kernels for models whose residual stream is kept in float32 whatever the compute dtype is,
// and whose norm comes after the sum (x <- norm(alpha x + y)):
//
//   asb_embedding_scaled      x[t] = table[id[t]] * scale, as float32
//   asb_cast_rows             float32 rows -> the compute dtype (what the next products read)
//   asb_scaled_add_rmsnorm    s = alpha x + y; out = gain * s / sqrt(mean(s^2) + eps), written as
//                             float32 (the stream) and/or in the compute dtype; optional row
//                             gather (the final norm of the rows whose logits are wanted)
//   asb_gated_rmsnorm         out = gain * o / sqrt(mean(o^2) + eps) * sigmoid(g), o float32,
//                             g a column range of a projection (a recurrent mixer's output gate)
//
// Sums, norms and gates are float32; each stored value is rounded once.
#include "common.cuh"
#include "gemm_partials.cuh"

namespace {

template <typename T>
__global__ void embedding_scaled_kernel(float* __restrict__ out, const T* __restrict__ table,
                                        const int* __restrict__ ids, int width, int vocab, float scale,
                                        int* __restrict__ status) {
  asb::pdl_wait();
  asb::pdl_launch_dependents();
  const int t = blockIdx.x;
  const int id = ids[t];
  float* dst = out + (size_t)t * width;
  if (id < 0 || id >= vocab) {  // refuse rather than read outside the table
    if (threadIdx.x == 0) atomicExch(status, 1);
    for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = 0.f;
    return;
  }
  const T* src = table + (size_t)id * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = asb::to_float(src[i]) * scale;
}

template <typename T>
__global__ void cast_rows_kernel(T* __restrict__ out, const float* __restrict__ in, long long total) {
  asb::pdl_wait();
  asb::pdl_launch_dependents();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x)
    out[i] = asb::from_float<T>(in[i]);
}

// One block per output row. y may be float32 or the compute dtype (TY), or absent.
template <typename T, typename TY>
__global__ void scaled_add_rmsnorm_kernel(float* __restrict__ out32, T* __restrict__ out_c,
                                          const float* __restrict__ x, const TY* __restrict__ y,
                                          const float* __restrict__ gain, const int* __restrict__ rows,
                                          int width, float alpha, float eps) {
  __shared__ float scratch[32];
  asb::pdl_wait();
  asb::pdl_launch_dependents();
  const size_t src = rows ? (size_t)rows[blockIdx.x] : (size_t)blockIdx.x;
  const float* xr = x + src * width;
  const TY* yr = y ? y + src * width : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float s = yr ? fmaf(alpha, xr[i], asb::to_float(yr[i])) : alpha * xr[i];
    ss = fmaf(s, s, ss);
  }
  const float inv = 1.f / sqrtf(asb::block_sum(ss, scratch) / (float)width + eps);
  const size_t dst = (size_t)blockIdx.x * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float s = yr ? fmaf(alpha, xr[i], asb::to_float(yr[i])) : alpha * xr[i];
    const float v = s * inv * gain[i];
    if (out32) out32[dst + i] = v;
    if (out_c) out_c[dst + i] = asb::from_float<T>(v);
  }
}

template <typename T>
__global__ void gated_rmsnorm_kernel(T* __restrict__ out, const float* __restrict__ o,
                                     const T* __restrict__ gate, int gate_stride,
                                     const float* __restrict__ gain, int width, float eps) {
  __shared__ float scratch[32];
  asb::pdl_wait();
  asb::pdl_launch_dependents();
  const float* row = o + (size_t)blockIdx.x * width;
  const T* g = gate + (size_t)blockIdx.x * gate_stride;
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) ss = fmaf(row[i], row[i], ss);
  const float inv = 1.f / sqrtf(asb::block_sum(ss, scratch) / (float)width + eps);
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float gv = asb::to_float(g[i]);
    out[(size_t)blockIdx.x * width + i] = asb::from_float<T>(row[i] * inv * gain[i] / (1.f + expf(-gv)));
  }
}

// The same with y given as the partial sums that the tensor-core GEMM left in its workspace (few
// tokens): a thread adds up the slots of 8 columns itself, so the GEMM's reduction kernel and a
// round trip of y through memory fall away. The slots are added in the reduction's order; only a
// row's squares are added in another order than in the kernel above (8 neighbouring columns a thread).
__global__ void partial_scaled_add_rmsnorm_kernel(float* __restrict__ out32, __nv_bfloat16* __restrict__ out_c,
                                                  const asb::PartialSums ps, const float* __restrict__ x,
                                                  const float* __restrict__ gain, int width, float alpha, float eps) {
  __shared__ float scratch[32];
  const int t = blockIdx.x, i = threadIdx.x * 8;
  const bool active = i < width;
  const int slots = active ? asb::partial_slots(ps, i / asb::kPartialRows) : 0;
  asb::pdl_wait();
  asb::pdl_launch_dependents();
  float v[8];
  float ss = 0.f;
  if (active) {
    float sum[8];
    asb::partial_sum<8>(ps, t, i, slots, sum);
    const float4 x0 = *reinterpret_cast<const float4*>(x + (size_t)t * width + i);
    const float4 x1 = *reinterpret_cast<const float4*>(x + (size_t)t * width + i + 4);
    const float xs[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      v[k] = fmaf(alpha, xs[k], sum[k]);
      ss = fmaf(v[k], v[k], ss);
    }
  }
  ss = asb::block_sum(ss, scratch);
  if (!active) return;
  const float inv = 1.f / sqrtf(ss / (float)width + eps);
  const float4 g0 = *reinterpret_cast<const float4*>(gain + i), g1 = *reinterpret_cast<const float4*>(gain + i + 4);
  const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
  uint4 packed;
  __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(&packed);
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    v[k] = v[k] * inv * g[k];
    o[k] = __float2bfloat16_rn(v[k]);
  }
  *reinterpret_cast<float4*>(out32 + (size_t)t * width + i) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(out32 + (size_t)t * width + i + 4) = make_float4(v[4], v[5], v[6], v[7]);
  *reinterpret_cast<uint4*>(out_c + (size_t)t * width + i) = packed;
}

int threads_for(int width) { return width >= 4096 ? 512 : (width >= 1024 ? 256 : 128); }

}  // namespace

extern "C" int asb_embedding_scaled(float* out, const void* table, const int* ids, int num_tokens, int width,
                                    int vocab, float scale, int dtype, int* status, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  ASB_DISPATCH_DTYPE(dtype, T, asb::launch(embedding_scaled_kernel<T>, num_tokens, threads_for(width), 0, stream, out,
                                           (const T*)table, ids, width, vocab, scale, status));
  return asb::check_launch("embedding_scaled");
}

extern "C" int asb_cast_rows(void* out, const float* in, long long total, int dtype, cudaStream_t stream) {
  if (total == 0) return 0;
  const long long blocks = (total + 255) / 256;
  ASB_DISPATCH_DTYPE(dtype, T, asb::launch(cast_rows_kernel<T>, (unsigned)(blocks < 148 * 16 ? blocks : 148 * 16), 256, 0,
                                           stream, (T*)out, in, total));
  return asb::check_launch("cast_rows");
}

// out32 and out_c: either may be null. y: null, float32 (y_dtype 0) or bfloat16 (1). rows: null or
// n source rows. dtype is that of out_c.
extern "C" int asb_scaled_add_rmsnorm(float* out32, void* out_c, const float* x, const void* y, int y_dtype,
                                      const float* gain, const int* rows, int n, int width, float alpha,
                                      float eps, int dtype, cudaStream_t stream) {
  if (n == 0) return 0;
  if (width < 1) return asb::fail("scaled_add_rmsnorm: width %d", width);
  const int threads = threads_for(width);
  ASB_DISPATCH_DTYPE(dtype, T, {
    if (y_dtype == asb::kFloat32)
      asb::launch(scaled_add_rmsnorm_kernel<T, float>, n, threads, 0, stream, out32, (T*)out_c, x, (const float*)y, gain,
                  rows, width, alpha, eps);
    else
      asb::launch(scaled_add_rmsnorm_kernel<T, __nv_bfloat16>, n, threads, 0, stream, out32, (T*)out_c, x,
                  (const __nv_bfloat16*)y, gain, rows, width, alpha, eps);
  });
  return asb::check_launch("scaled_add_rmsnorm");
}

extern "C" int asb_gated_rmsnorm(void* out, const float* o, const void* gate, int gate_stride, const float* gain,
                                 int n, int width, float eps, int dtype, cudaStream_t stream) {
  if (n == 0) return 0;
  ASB_DISPATCH_DTYPE(dtype, T, asb::launch(gated_rmsnorm_kernel<T>, n, threads_for(width), 0, stream, (T*)out, o,
                                           (const T*)gate, gate_stride, gain, width, eps));
  return asb::check_launch("gated_rmsnorm");
}

// out32 (float32) and out_c (bfloat16) = RMSNorm(alpha x + y), y being the partial sums of
// asb_gemm_tcgen05 mode 3 on [tokens, K] x [width, K]. Widths that are a multiple of 8 up to 8192,
// pointers 16-byte aligned.
extern "C" int asb_partial_scaled_add_rmsnorm(float* out32, void* out_c, const float* ws, int max_slots, int bn,
                                              int kb_per_tile, int num_tiles, int blocks, const float* x,
                                              const float* gain, int tokens, int width, float alpha, float eps,
                                              cudaStream_t stream) {
  if (tokens == 0) return 0;
  if (width % 8 || width / 8 > 1024) return asb::fail("partial_scaled_add_rmsnorm: width %d must be a multiple of 8 up to 8192", width);
  if (tokens > bn || num_tiles * asb::kPartialRows < width)
    return asb::fail("partial_scaled_add_rmsnorm: %d tokens x %d columns do not fit the partial sums (%d x %d)", tokens, width, bn,
                     num_tiles * asb::kPartialRows);
  if (((uintptr_t)out32 | (uintptr_t)out_c | (uintptr_t)x | (uintptr_t)gain | (uintptr_t)ws) & 15)
    return asb::fail("partial_scaled_add_rmsnorm: pointers must be 16-byte aligned");
  const asb::PartialSums ps = {ws, max_slots, bn, kb_per_tile, num_tiles, blocks};
  const int threads = ((width / 8) + 31) / 32 * 32;
  asb::launch(partial_scaled_add_rmsnorm_kernel, tokens, threads, 0, stream, out32, (__nv_bfloat16*)out_c, ps, x, gain, width,
              alpha, eps);
  return asb::check_launch("partial_scaled_add_rmsnorm");
}
