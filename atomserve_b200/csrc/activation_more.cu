// Further feed-forward activations, float32 inside and rounded once:
//
//   asb_gelu          out = 0.5 z (1 + erf(z / sqrt 2))            (tanh_form 0, the exact GELU)
//                     out = 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))       (tanh_form 1)
//                     out = max(z, 0)^2                            (tanh_form 2, the squared ReLU)
//   asb_clamped_glu   gu = [T, 2F], gate columns first: g = min(gate, limit),
//                     u = clamp(up, -limit, limit), out = g sigmoid(slope g) (u + shift)
//                     (limit <= 0: no clamping)
#include "common.cuh"

namespace asb {
__device__ __forceinline__ float gelu_erf(float z) { return 0.5f * z * (1.f + erff(z * 0.70710678118654752f)); }
__device__ __forceinline__ float gelu_tanh(float z) {
  return 0.5f * z * (1.f + tanhf(0.79788456080286536f * (z + 0.044715f * z * z * z)));
}
}  // namespace asb

namespace {

template <typename T>
__global__ void gelu_kernel(T* __restrict__ out, const T* __restrict__ in, long long total, int tanh_form) {
  asb::pdl_wait();
  asb::pdl_launch_dependents();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const float z = asb::to_float(in[i]);
    const float r = fmaxf(z, 0.f);
    out[i] = asb::from_float<T>(tanh_form == 2 ? r * r : (tanh_form ? asb::gelu_tanh(z) : asb::gelu_erf(z)));
  }
}

template <typename T>
__global__ void clamped_glu_kernel(T* __restrict__ out, const T* __restrict__ gu, int inter, long long total,
                                   float limit, float slope, float shift) {
  asb::pdl_wait();
  asb::pdl_launch_dependents();
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / inter;
    const int i = (int)(idx - t * inter);
    float g = asb::to_float(gu[t * 2 * inter + i]);
    float u = asb::to_float(gu[t * 2 * inter + inter + i]);
    if (limit > 0.f) {
      g = fminf(g, limit);
      u = fminf(fmaxf(u, -limit), limit);
    }
    out[idx] = asb::from_float<T>(g / (1.f + expf(-slope * g)) * (u + shift));
  }
}

unsigned grid_for(long long total) {
  const long long blocks = (total + 255) / 256;
  return (unsigned)(blocks < 148 * 32 ? blocks : 148 * 32);
}

}  // namespace

extern "C" int asb_gelu(void* out, const void* in, long long total, int tanh_form, int dtype, cudaStream_t stream) {
  if (total == 0) return 0;
  ASB_DISPATCH_DTYPE(dtype, T, asb::launch(gelu_kernel<T>, grid_for(total), 256, 0, stream, (T*)out, (const T*)in, total, tanh_form));
  return asb::check_launch("gelu");
}

extern "C" int asb_clamped_glu(void* out, const void* gate_up, int num_tokens, int inter, float limit, float slope,
                               float shift, int dtype, cudaStream_t stream) {
  if (num_tokens == 0 || inter == 0) return 0;
  const long long total = (long long)num_tokens * inter;
  ASB_DISPATCH_DTYPE(dtype, T, asb::launch(clamped_glu_kernel<T>, grid_for(total), 256, 0, stream, (T*)out,
                                           (const T*)gate_up, inter, total, limit, slope, shift));
  return asb::check_launch("clamped_glu");
}
