// The gated delta rule: a recurrent mixer with one matrix of state S [dk, dv] per head and request.
//
//   S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q            (in this order, per token)
//
// with q and k unit vectors per head (q also times dk^-1/2), both and v behind a short causal
// convolution over time and SiLU, beta = sigmoid(.), g = exp(-exp(A) softplus(a + dt)).  Everything
// behind the projections is float32.  A request's fixed-size state, one float32 vector per slot:
//   [ S of every head, stored [head][dv][dk] | the last taps-1 inputs of every convolved channel, [channel][taps-1] ].
//
// Four kernels per step:
//   delta_prepare      -- convolution (reading the slot's last inputs for the first tokens of an entry),
//                         SiLU, unit norms, beta and g, for all tokens in parallel;
//   delta_conv_carry   -- the slot's last taps-1 inputs after this step;
//   delta_recurrence   -- the recurrence, token by token within an entry, entries / heads / columns of S in parallel;
//   delta_output       -- per head o / rms(o) * w * silu(gate) in the activation dtype.
// Projection row (proj, [T, ldp]): q (G dk) | k (G dk) | v (H dv) | b (H) | a (H) | gate (H dv).
#include "common.cuh"

namespace srlm {

constexpr int kMaxTaps = 8;
constexpr int kLanesPerColumn = 8;       // lanes that share one column of S, each with every 8th row
constexpr int kColumnsPerBlock = 16;      // 16 x 8 lanes = 4 warps a block, one a scheduler: the recurrence is a chain

template <typename TP>
__global__ void delta_prepare_kernel(const TP* __restrict__ proj, long long ldp, const float* __restrict__ conv_w,
                                     const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                                     const float* __restrict__ state, long long state_stride,
                                     const int* __restrict__ entry_of_token, const int* __restrict__ cu_q,
                                     const int* __restrict__ slots, float* __restrict__ qkv_out,
                                     float* __restrict__ beta_out, float* __restrict__ decay_out,
                                     float* __restrict__ qk_out, int H, int G, int dk, int dv, int taps,
                                     float unit_eps) {
  pdl_wait();        // launched as a dependent of the kernel ahead: nothing is read before it has finished
  pdl_trigger();
  extern __shared__ float ch[];                              // [C] convolved and activated channels of this token
  const int t = blockIdx.x;
  const int C = 2 * G * dk + H * dv;
  const int e = entry_of_token[t];
  const int local = t - cu_q[e];                             // index of the token among the entry's tokens of this step
  const float* carry = state + (size_t)slots[e] * state_stride + (size_t)H * dk * dv;   // [C][taps - 1]
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float y = 0.f;
    for (int j = 0; j < taps; ++j) {
      const int back = taps - 1 - j;                         // the last column weighs the current token
      const float x = back <= local ? to_float(proj[(size_t)(t - back) * ldp + c])
                                    : carry[(size_t)c * (taps - 1) + (taps - 1) + (local - back)];
      y += conv_w[(size_t)c * taps + j] * x;
    }
    ch[c] = y / (1.f + expf(-y));
  }
  __syncthreads();
  // unit vectors: a warp per head of q and of k
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  for (int hh = warp; hh < 2 * G; hh += nwarps) {
    float* v = ch + (size_t)hh * dk;
    float ss = 0.f;
    for (int d = lane; d < dk; d += 32) ss += v[d] * v[d];
    ss = warp_sum(ss);
    float inv = 1.0f / sqrtf(ss + unit_eps);
    if (hh < G) inv *= 1.0f / sqrtf((float)dk);
    for (int d = lane; d < dk; d += 32) v[d] *= inv;
  }
  __syncthreads();
  for (int hh = warp; hh < G; hh += nwarps) {                // q . k of each q / k head: the same for every column of S
    float dot = 0.f;
    for (int d = lane; d < dk; d += 32) dot += ch[(size_t)hh * dk + d] * ch[(size_t)(G + hh) * dk + d];
    dot = warp_sum(dot);
    if (lane == 0) qk_out[(size_t)t * G + hh] = dot;
  }
  for (int c = threadIdx.x; c < C; c += blockDim.x) qkv_out[(size_t)t * C + c] = ch[c];
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    const float b = to_float(proj[(size_t)t * ldp + C + h]);
    const float a = to_float(proj[(size_t)t * ldp + C + H + h]) + dt_bias[h];
    const float sp = a > 20.f ? a : log1pf(expf(a));
    beta_out[(size_t)t * H + h] = 1.f / (1.f + expf(-b));
    decay_out[(size_t)t * H + h] = expf(-expf(a_log[h]) * sp);
  }
}

// One thread per (entry, channel): the last taps-1 inputs of the channel after this step, taken from the
// step's tokens and, where the step brought fewer than taps-1, from what the slot held.
template <typename TP>
__global__ void delta_conv_carry_kernel(const TP* __restrict__ proj, long long ldp, float* __restrict__ state,
                                        long long state_stride, long long carry_off, const int* __restrict__ cu_q,
                                        const int* __restrict__ slots, int n_entries, int C, int taps) {
  pdl_wait();        // launched as a dependent of the kernel ahead: nothing is read before it has finished
  pdl_trigger();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)n_entries * C) return;
  const int e = (int)(i / C), c = (int)(i % C);
  const int t0 = cu_q[e], n = cu_q[e + 1] - t0, keep = taps - 1;
  float* carry = state + (size_t)slots[e] * state_stride + carry_off + (size_t)c * keep;
  float fresh[kMaxTaps];
#pragma unroll
  for (int k = 0; k < kMaxTaps; ++k) {
    if (k >= keep) break;
    const int rel = n - keep + k;                            // index among the step's tokens; negative: held before
    fresh[k] = rel >= 0 ? to_float(proj[(size_t)(t0 + rel) * ldp + c]) : carry[keep + rel];
  }
#pragma unroll
  for (int k = 0; k < kMaxTaps; ++k) {
    if (k >= keep) break;
    carry[k] = fresh[k];
  }
}

// Block: 16 columns of one head's S for one entry; a column is shared by 8 lanes, lane l holding rows
// 32 j + 4 l + {0..3} (RPL of them, four consecutive at a time so that shared memory is read 16 bytes a
// lane).  The entry's tokens come through shared memory in chunks of 16, the next chunk fetched (cp.async)
// while this one is worked on.  Per token the dependent chain is one round of partial sums over the OLD
// state and one round of shuffles: with a = k . S and b = q . S (both over the state before the token)
// and c = q . k (the same for every column: delta_prepare forms it),
//     u = beta (v - g a),   S <- g S + k u,   o = g b + c u      ( = q . S after the write )
// so the two sums are reduced side by side and the state update is one FMA deep.
constexpr int kChunk = 16;

__device__ __forceinline__ void cp_async_4(float* dst, const float* src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src));
}

template <int RPL>
__global__ void __launch_bounds__(kColumnsPerBlock* kLanesPerColumn)
delta_recurrence_kernel(const float* __restrict__ qkv, const float* __restrict__ beta, const float* __restrict__ decay,
                        const float* __restrict__ qk, float* __restrict__ state, long long state_stride, const int* __restrict__ cu_q,
                        const int* __restrict__ slots, float* __restrict__ o_out, int H, int G, int dk, int dv) {
  pdl_wait();        // launched as a dependent of the kernel ahead: nothing is read before it has finished
  pdl_trigger();
  constexpr int DKP = RPL * kLanesPerColumn;                 // rows held in shared memory (zero beyond dk)
  constexpr int ROW = 2 * DKP + kColumnsPerBlock + 4;        // k | q | v of the block's columns | beta, g, q.k, -
  extern __shared__ __align__(16) float stage[];            // [2][kChunk][ROW]
  const int e = blockIdx.z, h = blockIdx.y;
  const int cg = threadIdx.x / kLanesPerColumn, l = threadIdx.x % kLanesPerColumn;
  const int col = blockIdx.x * kColumnsPerBlock + cg;
  const bool live = col < dv;
  const int kh = h / (H / G);
  const int C = 2 * G * dk + H * dv;
  const int t0 = cu_q[e], n_tok = cu_q[e + 1] - t0;
  float* S_col = state + (size_t)slots[e] * state_stride + ((size_t)h * dv + (live ? col : 0)) * dk;
  float S[RPL];
#pragma unroll
  for (int i = 0; i < RPL; ++i) {
    const int r = (i >> 2) * 32 + 4 * l + (i & 3);
    S[i] = (live && r < dk) ? S_col[r] : 0.f;
  }
  for (int idx = threadIdx.x; idx < 2 * kChunk * ROW; idx += blockDim.x) stage[idx] = 0.f;
  __syncthreads();
  const int col0 = blockIdx.x * kColumnsPerBlock;
  auto fetch = [&](int chunk, int buf) {
    const int base = chunk * kChunk, n = min(kChunk, n_tok - base);
    float* st = stage + buf * kChunk * ROW;
    for (int idx = threadIdx.x; idx < n * dk; idx += blockDim.x) {
      const int i = idx / dk, r = idx - i * dk;
      const float* row = qkv + (size_t)(t0 + base + i) * C;
      cp_async_4(st + i * ROW + r, row + (size_t)(G + kh) * dk + r);            // k
      cp_async_4(st + i * ROW + DKP + r, row + (size_t)kh * dk + r);            // q
    }
    for (int idx = threadIdx.x; idx < n * kColumnsPerBlock; idx += blockDim.x) {
      const int i = idx / kColumnsPerBlock, c = idx - i * kColumnsPerBlock;
      if (col0 + c < dv)
        cp_async_4(st + i * ROW + 2 * DKP + c, qkv + (size_t)(t0 + base + i) * C + 2 * G * dk + (size_t)h * dv + col0 + c);
    }
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      cp_async_4(st + i * ROW + 2 * DKP + kColumnsPerBlock, beta + (size_t)(t0 + base + i) * H + h);
      cp_async_4(st + i * ROW + 2 * DKP + kColumnsPerBlock + 1, decay + (size_t)(t0 + base + i) * H + h);
      cp_async_4(st + i * ROW + 2 * DKP + kColumnsPerBlock + 2, qk + (size_t)(t0 + base + i) * G + kh);
    }
    asm volatile("cp.async.commit_group;" ::);
  };
  const int chunks = (n_tok + kChunk - 1) / kChunk;
  if (chunks > 0) fetch(0, 0);
  for (int c = 0; c < chunks; ++c) {
    const int buf = c & 1;
    if (c + 1 < chunks) {
      fetch(c + 1, buf ^ 1);
      asm volatile("cp.async.wait_group 1;" ::);
    } else {
      asm volatile("cp.async.wait_group 0;" ::);
    }
    __syncthreads();
    const float* st = stage + buf * kChunk * ROW;
    const int n = min(kChunk, n_tok - c * kChunk);
    for (int i = 0; i < n; ++i) {
      const float* row = st + i * ROW;
      float kk[RPL], qq[RPL];
#pragma unroll
      for (int j = 0; j < RPL / 4; ++j) {
        const float4 kv = *reinterpret_cast<const float4*>(row + j * 32 + 4 * l);
        const float4 qv = *reinterpret_cast<const float4*>(row + DKP + j * 32 + 4 * l);
        kk[4 * j] = kv.x; kk[4 * j + 1] = kv.y; kk[4 * j + 2] = kv.z; kk[4 * j + 3] = kv.w;
        qq[4 * j] = qv.x; qq[4 * j + 1] = qv.y; qq[4 * j + 2] = qv.z; qq[4 * j + 3] = qv.w;
      }
      const float v = row[2 * DKP + cg], bt = row[2 * DKP + kColumnsPerBlock], g = row[2 * DKP + kColumnsPerBlock + 1];
      const float cc = row[2 * DKP + kColumnsPerBlock + 2];
      float a4[4] = {0.f, 0.f, 0.f, 0.f}, b4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int j = 0; j < RPL; ++j) {                        // four running sums each: no chain of RPL additions
        a4[j & 3] += kk[j] * S[j];
        b4[j & 3] += qq[j] * S[j];
      }
      float a = (a4[0] + a4[1]) + (a4[2] + a4[3]), b = (b4[0] + b4[1]) + (b4[2] + b4[3]);
#pragma unroll
      for (int off = 1; off < kLanesPerColumn; off <<= 1) {
        a += __shfl_xor_sync(0xffffffffu, a, off);
        b += __shfl_xor_sync(0xffffffffu, b, off);
      }
      const float u = bt * (v - g * a);
#pragma unroll
      for (int j = 0; j < RPL; ++j) S[j] = g * S[j] + kk[j] * u;
      if (live && l == 0) o_out[((size_t)(t0 + c * kChunk + i) * H + h) * dv + col] = g * b + cc * u;
    }
    __syncthreads();                                         // the chunk is done with before its buffer is fetched into
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < RPL; ++i) {
      const int r = (i >> 2) * 32 + 4 * l + (i & 3);
      if (r < dk) S_col[r] = S[i];
    }
  }
}

// One block per token, a warp per head: o / sqrt(mean(o^2) + eps) * w * silu(gate).
template <typename TP, typename TA>
__global__ void delta_output_kernel(const float* __restrict__ o, const float* __restrict__ norm_w, float eps,
                                    const TP* __restrict__ proj, long long ldp, int gate_off, TA* __restrict__ out,
                                    int H, int dv) {
  pdl_wait();        // launched as a dependent of the kernel ahead: nothing is read before it has finished
  pdl_trigger();
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  for (int h = warp; h < H; h += nwarps) {
    const float* row = o + ((size_t)t * H + h) * dv;
    float ss = 0.f;
    for (int d = lane; d < dv; d += 32) ss += row[d] * row[d];
    const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)dv + eps);
    for (int d = lane; d < dv; d += 32) {
      const float z = to_float(proj[(size_t)t * ldp + gate_off + (size_t)h * dv + d]);
      out[((size_t)t * H + h) * dv + d] = from_float<TA>(row[d] * inv * norm_w[d] * (z / (1.f + expf(-z))));
    }
  }
}

}  // namespace srlm

using namespace srlm;

static int delta_sizes_ok(int H, int G, int dk, int dv, int taps) {
  return H > 0 && G > 0 && H % G == 0 && dk > 0 && dk <= 512 && dv > 0 && taps >= 1 && taps <= kMaxTaps;
}

extern "C" int srlm_delta_prepare(const void* proj, int proj_dtype, long long ldp, const float* conv_w,
                                  const float* a_log, const float* dt_bias, float* state, long long state_stride,
                                  const int* entry_of_token, const int* cu_q, const int* slots, int n_entries,
                                  float* qkv_out, float* beta_out, float* decay_out, float* qk_out, int T, int H,
                                  int G, int dk, int dv, int taps, float unit_eps, cudaStream_t stream) {
  if (T <= 0) return ST_OK;
  const long long C = 2LL * G * dk + (long long)H * dv;
  if (!delta_sizes_ok(H, G, dk, dv, taps) || ldp < C + 2LL * H + (long long)H * dv || C * 4 > 200 * 1024 ||
      state_stride < (long long)H * dk * dv + C * (taps - 1))
    return refuse(ST_BAD_SIZE, "delta_prepare: H=%d G=%d dk=%d dv=%d taps=%d ldp=%lld state=%lld (dk <= 512, taps <= %d)",
                  H, G, dk, dv, taps, ldp, state_stride, kMaxTaps);
  const size_t smem = (size_t)C * sizeof(float);
  SRLM_DISPATCH_ACT(proj_dtype, TP, {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(delta_prepare_kernel<TP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_pdl(delta_prepare_kernel<TP>, dim3(T), dim3(256), smem, stream, (const TP*)proj, ldp, conv_w, a_log, dt_bias, state, state_stride,
                                                       entry_of_token, cu_q, slots, qkv_out, beta_out, decay_out, qk_out,
                                                       H, G, dk, dv, taps, unit_eps);
    if (taps > 1) {
      const long long n = (long long)n_entries * C;
      launch_pdl(delta_conv_carry_kernel<TP>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, 
          (const TP*)proj, ldp, state, state_stride, (long long)H * dk * dv, cu_q, slots, n_entries, (int)C, taps);
    }
  });
  return launched();
}

extern "C" int srlm_delta_recurrence(const float* qkv, const float* beta, const float* decay, const float* qk, float* state,
                                     long long state_stride, const int* cu_q, const int* slots, int n_entries,
                                     float* o_out, int H, int G, int dk, int dv, cudaStream_t stream) {
  if (n_entries <= 0) return ST_OK;
  if (!delta_sizes_ok(H, G, dk, dv, 1) || n_entries > 65535 || H > 65535)
    return refuse(ST_BAD_SIZE, "delta_recurrence: H=%d G=%d dk=%d dv=%d entries=%d (dk <= 512)", H, G, dk, dv, n_entries);
  dim3 grid((dv + kColumnsPerBlock - 1) / kColumnsPerBlock, H, n_entries);
  const int threads = kColumnsPerBlock * kLanesPerColumn;
  const int rpl = (dk + kLanesPerColumn - 1) / kLanesPerColumn;
#define SRLM_DELTA_CASE(R)                                                                                       \
  do {                                                                                                           \
    const size_t smem = (size_t)2 * kChunk * (2 * R * kLanesPerColumn + kColumnsPerBlock + 4) * sizeof(float);   \
    if (smem > 48 * 1024)                                                                                        \
      cudaFuncSetAttribute(delta_recurrence_kernel<R>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
    launch_pdl(delta_recurrence_kernel<R>, dim3(grid), dim3(threads), smem, stream, qkv, beta, decay, qk, state, state_stride, cu_q, \
                                                                slots, o_out, H, G, dk, dv);                     \
  } while (0)
  if (rpl <= 4) SRLM_DELTA_CASE(4);
  else if (rpl <= 8) SRLM_DELTA_CASE(8);
  else if (rpl <= 16) SRLM_DELTA_CASE(16);
  else if (rpl <= 32) SRLM_DELTA_CASE(32);
  else SRLM_DELTA_CASE(64);     // heads of up to 512: the state no longer fits the registers, and runs from local memory
#undef SRLM_DELTA_CASE
  return launched();
}

extern "C" int srlm_delta_output(const float* o, const float* norm_w, float eps, const void* proj, int proj_dtype,
                                 long long ldp, int gate_off, void* out, int out_dtype, int T, int H, int dv,
                                 cudaStream_t stream) {
  if (T <= 0) return ST_OK;
  if (H <= 0 || dv <= 0 || !(eps > 0.f) || gate_off < 0 || ldp < gate_off + (long long)H * dv)
    return refuse(ST_BAD_SIZE, "delta_output: H=%d dv=%d gate_off=%d ldp=%lld", H, dv, gate_off, ldp);
  const int threads = 32 * (H < 8 ? H : 8);
#define SRLM_DELTA_OUT(TP, TA)                                                                                    \
  launch_pdl(delta_output_kernel<TP, TA>, dim3(T), dim3(threads), 0, stream, o, norm_w, eps, (const TP*)proj, ldp, gate_off, (TA*)out, H, dv)
  if (proj_dtype == DT_F32 && out_dtype == DT_F32) SRLM_DELTA_OUT(float, float);
  else if (proj_dtype == DT_F32 && out_dtype == DT_BF16) SRLM_DELTA_OUT(float, bf16);
  else if (proj_dtype == DT_BF16 && out_dtype == DT_BF16) SRLM_DELTA_OUT(bf16, bf16);
  else return refuse(ST_BAD_DTYPE, "delta_output: projection dtype %d with output dtype %d", proj_dtype, out_dtype);
#undef SRLM_DELTA_OUT
  return launched();
}
