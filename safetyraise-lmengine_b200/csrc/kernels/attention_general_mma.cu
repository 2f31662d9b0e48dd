// The attention of attention_general.cu on bfloat16 tensor cores (mma.sync m16n8k16, float32 sums),
// for steps with many rows (prompts and their portions): keys of dk and values of dv elements, values
// optionally read from the keys' leading part, an optional sink per head.
//
// A block of four warps takes 64 rows (tokens x query heads of one KV head) of one entry and one slab of
// DVT = 64 or 128 value columns, and walks the keys in tiles of 64: S = Q K^T over the whole key size, the
// softmax in registers (float32), O += P V for the block's slab.  A wide value (a latent of 512) is cut
// into slabs with a block each, every block forming S again: the sums of 64 rows x 512 columns do not
// fit a block's registers, and S costs less on tensor cores than it did in float32 arithmetic.
// Queries arrive as float32 and are rounded to bfloat16 as they enter shared memory.
#include <math_constants.h>

#include "common.cuh"

namespace srlm {

constexpr int kMmaRows = 64, kMmaKeys = 64, kMmaWarps = 4, kPad = 8;

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const bf16* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const bf16* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <typename TO, int NT>       // NT: 8-column tiles of the block's slab of values (8 or 16)
__global__ void __launch_bounds__(kMmaWarps * 32)
paged_attention_general_mma_kernel(const float* __restrict__ q, const bf16* __restrict__ k_cache,
                                   const bf16* __restrict__ v_cache, TO* __restrict__ out,
                                   const int* __restrict__ block_table, int table_stride,
                                   const int* __restrict__ cu_q, const int* __restrict__ kv_lens,
                                   const float* __restrict__ sinks, int nq, int nkv, int dk, int dv, int page_size,
                                   float scale, int window) {
  constexpr int DVT = 8 * NT;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int slabs = dv / DVT;
  const int e = blockIdx.z, kvh = blockIdx.y / slabs, slab = blockIdx.y % slabs;
  const int G = nq / nkv;
  const int t0 = cu_q[e], q_len = cu_q[e + 1] - t0, kv_len = kv_lens[e];
  const int rows = q_len * G;
  const int r0 = blockIdx.x * kMmaRows;
  if (r0 >= rows) return;
  const int ks = dk + kPad;                                 // row strides in elements; rows stay 16-byte aligned
  const int vs = v_cache ? DVT + kPad : ks;
  bf16* q_s = reinterpret_cast<bf16*>(smem_raw);            // [64][dk + 8]
  bf16* k_s = q_s + kMmaRows * ks;                          // [64][dk + 8]
  bf16* v_s = v_cache ? k_s + kMmaKeys * ks : k_s + slab * DVT;   // [64][DVT + 8], or the slab's columns of the keys
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int start = kv_len - q_len;
  const int* table = block_table + (size_t)e * table_stride;

  for (int idx = tid; idx < kMmaRows * dk; idx += blockDim.x) {
    const int r = idx / dk, d = idx - r * dk, row = r0 + r;
    const float v = row < rows ? q[((size_t)(t0 + row / G) * nq + kvh * G + row % G) * dk + d] : 0.f;
    q_s[r * ks + d] = __float2bfloat16_rn(v);
  }

  // a thread's two rows of its warp's 16: lane / 4 and lane / 4 + 8
  float m[2], l[2];
  int pos[2], first[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = r0 + warp * 16 + (lane >> 2) + 8 * i;
    const bool live = row < rows;
    pos[i] = live ? start + row / G : -1;
    first[i] = (window > 0 && live) ? max(0, pos[i] - window + 1) : 0;
    const int h = kvh * G + (live ? row % G : 0);
    m[i] = sinks ? sinks[h] : -CUDART_INF_F;
    l[i] = sinks ? 1.f : 0.f;
  }
  float o[NT][4];
#pragma unroll
  for (int n = 0; n < NT; ++n)
#pragma unroll
    for (int c = 0; c < 4; ++c) o[n][c] = 0.f;

  const int last_row = min(rows, r0 + kMmaRows) - 1;
  const int max_pos = start + last_row / G, min_pos = start + r0 / G;
  const int first_key = window > 0 ? max(0, min_pos - window + 1) : 0;
  const int kvec = dk / 8, vvec = DVT / 8;

  for (int jb = (first_key / kMmaKeys) * kMmaKeys; jb <= max_pos; jb += kMmaKeys) {
    __syncthreads();
    for (int idx = tid; idx < kMmaKeys * kvec; idx += blockDim.x) {
      const int jj = idx / kvec, c = idx - jj * kvec, j = jb + jj;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (j <= max_pos) {
        const size_t rowi = ((size_t)table[j / page_size] * nkv + kvh) * page_size + (j % page_size);
        v = *reinterpret_cast<const uint4*>(k_cache + rowi * dk + c * 8);
      }
      *reinterpret_cast<uint4*>(k_s + jj * ks + c * 8) = v;
    }
    if (v_cache) {
      for (int idx = tid; idx < kMmaKeys * vvec; idx += blockDim.x) {
        const int jj = idx / vvec, c = idx - jj * vvec, j = jb + jj;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (j <= max_pos) {
          const size_t rowi = ((size_t)table[j / page_size] * nkv + kvh) * page_size + (j % page_size);
          v = *reinterpret_cast<const uint4*>(v_cache + rowi * dv + slab * DVT + c * 8);
        }
        *reinterpret_cast<uint4*>(v_s + jj * vs + c * 8) = v;
      }
    }
    __syncthreads();

    // S = Q K^T: 16 rows x 64 keys a warp
    float s[8][4];
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
      for (int c = 0; c < 4; ++c) s[n][c] = 0.f;
    const bf16* qa = q_s + (warp * 16 + (lane & 15)) * ks + (lane >> 4) * 8;
    const bf16* kb = k_s + ((lane & 7) + (lane >> 4) * 8) * ks + ((lane >> 3) & 1) * 8;
    for (int k0 = 0; k0 < dk; k0 += 16) {
      uint32_t a[4];
      ldmatrix_x4(a, qa + k0);
#pragma unroll
      for (int n2 = 0; n2 < 4; ++n2) {
        uint32_t b[4];
        ldmatrix_x4(b, kb + n2 * 16 * ks + k0);
        mma_bf16(s[2 * n2], a, b[0], b[1]);
        mma_bf16(s[2 * n2 + 1], a, b[2], b[3]);
      }
    }

    // softmax of this tile, in registers
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      float mx = -CUDART_INF_F;
#pragma unroll
      for (int n = 0; n < 8; ++n)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int j = jb + n * 8 + (lane & 3) * 2 + c;
          const bool valid = j <= pos[i] && j >= first[i];
          const float v = valid ? s[n][2 * i + c] * scale : -CUDART_INF_F;
          s[n][2 * i + c] = v;
          mx = fmaxf(mx, v);
        }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m[i], mx);
      float alpha = 1.f, sum = 0.f;
      if (m_new != -CUDART_INF_F) {
        alpha = expf(m[i] - m_new);
#pragma unroll
        for (int n = 0; n < 8; ++n)
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const float p = expf(s[n][2 * i + c] - m_new);       // exp(-inf) = 0 for masked keys
            s[n][2 * i + c] = p;
            sum += p;
          }
      } else {
#pragma unroll
        for (int n = 0; n < 8; ++n) s[n][2 * i] = s[n][2 * i + 1] = 0.f;
      }
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      l[i] = l[i] * alpha + sum;
      m[i] = m_new;
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        o[n][2 * i] *= alpha;
        o[n][2 * i + 1] *= alpha;
      }
    }

    // O += P V for the slab
    const bf16* vb = v_s + (lane & 15) * vs + (lane >> 4) * 8;
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      uint32_t a[4];
      a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
      a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int n2 = 0; n2 < NT / 2; ++n2) {
        uint32_t b[4];
        ldmatrix_x4_trans(b, vb + kk * 16 * vs + n2 * 16);
        mma_bf16(o[2 * n2], a, b[0], b[1]);
        mma_bf16(o[2 * n2 + 1], a, b[2], b[3]);
      }
    }
  }

#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = r0 + warp * 16 + (lane >> 2) + 8 * i;
    if (row >= rows) continue;
    const float inv = 1.f / l[i];
    TO* dst = out + ((size_t)(t0 + row / G) * nq + kvh * G + row % G) * dv + slab * DVT + (lane & 3) * 2;
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      dst[n * 8] = from_float<TO>(o[n][2 * i] * inv);
      dst[n * 8 + 1] = from_float<TO>(o[n][2 * i + 1] * inv);
    }
  }
}

template <typename TO, int NT>
static int launch_mma(dim3 grid, size_t smem, cudaStream_t stream, const float* q, const void* k_cache,
                      const void* v_cache, void* out, const int* block_table, int table_stride, const int* cu_q,
                      const int* kv_lens, const float* sinks, int nq, int nkv, int dk, int dv, int page_size,
                      float scale, int window) {
  auto kern = paged_attention_general_mma_kernel<TO, NT>;
  if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  kern<<<grid, kMmaWarps * 32, smem, stream>>>(q, (const bf16*)k_cache, (const bf16*)v_cache, (TO*)out, block_table,
                                               table_stride, cu_q, kv_lens, sinks, nq, nkv, dk, dv, page_size, scale,
                                               window);
  return launched();
}

}  // namespace srlm

using namespace srlm;

// Whether the tensor-core form takes these sizes: key size a multiple of 16, value size a multiple of 64,
// and two tiles of 64 rows of the key size within a block's shared memory.
extern "C" int srlm_attention_general_mma_takes(int dk, int dv, int values_from_keys) {
  if (dk <= 0 || dv <= 0 || dk % 16 || dv % 64 || (values_from_keys && dv > dk)) return 0;
  const size_t slab = dv % 128 == 0 ? 128 : 64;
  const size_t smem = (size_t)2 * kMmaRows * (dk + kPad) * 2 + (values_from_keys ? 0 : kMmaKeys * (slab + kPad) * 2);
  return smem <= 220 * 1024 ? 1 : 0;
}

// The contract of srlm_paged_attention_general for a bfloat16 cache, without key slices.
extern "C" int srlm_paged_attention_general_mma(const float* q, const void* k_cache, const void* v_cache, void* out,
                                                int out_dtype, const int* block_table, int table_stride,
                                                const int* cu_q, const int* kv_lens, const float* sinks,
                                                int n_entries, int max_q_len, int nq, int nkv, int dk, int dv,
                                                int page_size, float scale, int window, cudaStream_t stream) {
  if (n_entries <= 0 || max_q_len <= 0) return ST_OK;
  if (nq <= 0 || nkv <= 0 || nq % nkv || page_size <= 0 || !srlm_attention_general_mma_takes(dk, dv, v_cache ? 0 : 1))
    return refuse(ST_BAD_SIZE, "paged_attention_general_mma: nq=%d nkv=%d dk=%d dv=%d page_size=%d (dk a multiple of "
                  "16, dv of 64)", nq, nkv, dk, dv, page_size);
  if ((((uintptr_t)k_cache | (uintptr_t)v_cache) & 15) != 0)
    return refuse(ST_BAD_ALIGN, "paged_attention_general_mma: the pools must be 16-byte aligned");
  const int slab = dv % 128 == 0 ? 128 : 64;
  const int G = nq / nkv;
  const long long tiles = ((long long)max_q_len * G + kMmaRows - 1) / kMmaRows;
  const long long y = (long long)nkv * (dv / slab);
  if (n_entries > 65535 || y > 65535) return refuse(ST_BAD_SIZE, "paged_attention_general_mma: %d entries", n_entries);
  dim3 grid((unsigned)tiles, (unsigned)y, (unsigned)n_entries);
  const size_t smem = (size_t)2 * kMmaRows * (dk + kPad) * 2 + (v_cache ? (size_t)kMmaKeys * (slab + kPad) * 2 : 0);
#define SRLM_MMA_ARGS grid, smem, stream, q, k_cache, v_cache, out, block_table, table_stride, cu_q, kv_lens, sinks, nq, \
                      nkv, dk, dv, page_size, scale, window
  if (out_dtype == DT_F32) return slab == 128 ? launch_mma<float, 16>(SRLM_MMA_ARGS) : launch_mma<float, 8>(SRLM_MMA_ARGS);
  if (out_dtype == DT_BF16) return slab == 128 ? launch_mma<bf16, 16>(SRLM_MMA_ARGS) : launch_mma<bf16, 8>(SRLM_MMA_ARGS);
#undef SRLM_MMA_ARGS
  return refuse(ST_BAD_DTYPE, "paged_attention_general_mma: output dtype %d", out_dtype);
}
