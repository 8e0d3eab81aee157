// Kernels of a block whose branches read the same residual stream (sm_100a), float32 and bfloat16.
//
//   add_scaled_rmsnorm: v = h[t] + sa * a[t] + sb * b[t] (sa, sb vectors over the width, each term optional);
//                       if write_h: h[t] = v;  y1[r] = v * rsqrt(mean(v^2) + eps) * g1;  y2[r] = ... * g2 (optional).
//                       Rows: r = 0..R-1, t = rows ? rows[r] : r.  One block a row; the row stays in shared memory
//                       between the sum of squares and the outputs, so memory is passed over once.
//   add_scaled:         h[t] += sa * a[t] + sb * b[t]        (no norm behind it)
//   scale_rows:         x *= s                               (float32, in place: logits)
// The stream, the factors, the gains and all sums are 32-bit; a and b may each be float32 or bfloat16.
#include "common.cuh"

__device__ __forceinline__ float ld_any(const void* p, int dt, size_t i) {
  return dt == SX_F32 ? ((const float*)p)[i] : __bfloat162float(((const bf16*)p)[i]);
}

template <typename TO>
__global__ void __launch_bounds__(256) add_scaled_rmsnorm_kernel(
    float* __restrict__ h, const void* __restrict__ a, int a_dt, const float* __restrict__ sa,
    const void* __restrict__ b, int b_dt, const float* __restrict__ sb, const float* __restrict__ g1,
    const float* __restrict__ g2, float eps, TO* __restrict__ y1, TO* __restrict__ y2, const int* __restrict__ rows,
    int H, int write_h) {
  extern __shared__ float row[];
  __shared__ float red[33];
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x;
  const int t = rows ? rows[r] : r;
  float* hr = h + (size_t)t * H;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = hr[i];
    if (a || b) {
      float d = 0.f;
      if (a) d = ld_any(a, a_dt, (size_t)t * H + i) * (sa ? sa[i] : 1.f);
      if (b) d += ld_any(b, b_dt, (size_t)t * H + i) * (sb ? sb[i] : 1.f);
      v += d;
      if (write_h) hr[i] = v;
    }
    row[i] = v;
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float v = row[i] * inv;
    y1[(size_t)r * H + i] = from_f32<TO>(v * g1[i]);
    if (y2) y2[(size_t)r * H + i] = from_f32<TO>(v * g2[i]);
  }
}

extern "C" int sx_add_scaled_rmsnorm(float* h, const void* a, int a_dt, const float* sa, const void* b, int b_dt,
                                     const float* sb, const float* g1, const float* g2, float eps, void* y1, void* y2,
                                     const int* rows, int R, int H, int out_dt, int write_h, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (H <= 0 || H > 24576) return SX_ERR_SIZE;
  const size_t smem = (size_t)H * sizeof(float);
  if (out_dt == SX_F32) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(add_scaled_rmsnorm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return sx_launch(add_scaled_rmsnorm_kernel<float>, dim3(R), dim3(256), smem, stream, h, a, a_dt, sa, b, b_dt, sb, g1, g2,
                     eps, (float*)y1, (float*)y2, rows, H, write_h);
  }
  if (out_dt == SX_BF16) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(add_scaled_rmsnorm_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return sx_launch(add_scaled_rmsnorm_kernel<bf16>, dim3(R), dim3(256), smem, stream, h, a, a_dt, sa, b, b_dt, sb, g1, g2,
                     eps, (bf16*)y1, (bf16*)y2, rows, H, write_h);
  }
  return SX_ERR_DTYPE;
}

__global__ void add_scaled_kernel(float* __restrict__ h, const void* __restrict__ a, int a_dt, const float* __restrict__ sa,
                                  const void* __restrict__ b, int b_dt, const float* __restrict__ sb, int H, size_t n) {
  pdl_wait();
  pdl_trigger();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int c = (int)(i % H);
  float d = 0.f;
  if (a) d = ld_any(a, a_dt, i) * (sa ? sa[c] : 1.f);
  if (b) d += ld_any(b, b_dt, i) * (sb ? sb[c] : 1.f);
  h[i] += d;
}

extern "C" int sx_add_scaled(float* h, const void* a, int a_dt, const float* sa, const void* b, int b_dt, const float* sb,
                             int T, int H, cudaStream_t stream) {
  if (T <= 0 || H <= 0) return 0;
  const size_t n = (size_t)T * H;
  return sx_launch(add_scaled_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, h, a, a_dt, sa, b, b_dt, sb, H, n);
}

__global__ void scale_rows_kernel(float* __restrict__ x, float s, size_t n) {
  pdl_wait();
  pdl_trigger();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) x[i] *= s;
}

extern "C" int sx_scale_rows(float* x, long long n, float s, cudaStream_t stream) {
  if (n <= 0) return 0;
  return sx_launch(scale_rows_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, x, s, (size_t)n);
}
