// A sublayer's result on its way into the residual stream of a block that norms on both sides:
//
//   y        = sub * sigmoid(gate + gate_bias)            (gate: the logits of a learned gate; optional)
//   residual = residual + post_w * y / sqrt(mean(y^2) + eps)
//   next_out = next_w * residual / sqrt(mean(residual^2) + next_eps)   (optional: the norm ahead of the next sublayer)
//
// One block per token, the row kept in shared memory between the passes, every sum in float32 in an
// order fixed by the width.  post_w is a vector (a norm with one number repeats it).
#include "common.cuh"

namespace srlm {

template <typename TA>
__global__ void gated_postnorm_add_kernel(float* __restrict__ residual, const TA* __restrict__ sub,
                                          const TA* __restrict__ gate, const float* __restrict__ gate_bias,
                                          const float* __restrict__ post_w, float eps,
                                          const float* __restrict__ next_w, float next_eps, TA* __restrict__ next_out,
                                          int H) {
  pdl_wait();        // launched as a dependent of the kernel ahead: nothing is read before it has finished
  pdl_trigger();
  extern __shared__ float row[];
  __shared__ float scratch[32];
  const size_t base = (size_t)blockIdx.x * H;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float y = to_float(sub[base + i]);
    if (gate) {
      const float z = to_float(gate[base + i]) + (gate_bias ? gate_bias[i] : 0.f);
      y *= 1.f / (1.f + expf(-z));
    }
    row[i] = y;
    ss += y * y;
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)H + eps);
  float ss2 = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float x = residual[base + i] + row[i] * inv * post_w[i];
    residual[base + i] = x;
    row[i] = x;
    ss2 += x * x;
  }
  if (!next_out) return;
  const float inv2 = 1.0f / sqrtf(block_sum(ss2, scratch) / (float)H + next_eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x) next_out[base + i] = from_float<TA>(row[i] * inv2 * next_w[i]);
}

}  // namespace srlm

using namespace srlm;

extern "C" int srlm_gated_postnorm_add(float* residual, const void* sub, const void* gate, const float* gate_bias,
                                       const float* post_w, float eps, const float* next_w, float next_eps,
                                       void* next_out, int act_dtype, int T, int H, cudaStream_t stream) {
  if (T <= 0) return ST_OK;
  if (H <= 0 || !(eps > 0.f) || !post_w || (next_out && (!next_w || !(next_eps > 0.f))))
    return refuse(ST_BAD_SIZE, "gated_postnorm_add: H=%d eps=%g next_eps=%g", H, (double)eps, (double)next_eps);
  const size_t smem = (size_t)H * sizeof(float);
  if (smem > 200 * 1024) return refuse(ST_BAD_SIZE, "gated_postnorm_add: a row of %d elements does not fit", H);
  int block = 64;
  while (block < 1024 && block * 4 < H) block <<= 1;
  SRLM_DISPATCH_ACT(act_dtype, TA, {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(gated_postnorm_add_kernel<TA>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_pdl(gated_postnorm_add_kernel<TA>, dim3(T), dim3(block), smem, stream, residual, (const TA*)sub, (const TA*)gate, gate_bias,
                                                              post_w, eps, next_w, next_eps, (TA*)next_out, H);
  });
  return launched();
}
