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
