// Latent attention on CUDA cores, float32 arithmetic, any sizes: the true 32-bit path of the mixer and
// the path that takes every geometry in bfloat16 when the tensor-core kernel refuses one.
//
// The mixer keeps, per token, one row [c | kr] of R + dr numbers: c = the RMS-normed latent of keys and
// values, kr = the rotated key part that all heads share. With k_h = Wk_h c and v_h = Wv_h c,
//   score_h(i, j) = (qn_h(i) . Wk_h c(j) + qr_h(i) . kr(j)) * scale = ([Wk_h^T qn_h(i) | qr_h(i)] . [c(j) | kr(j)]) * scale
//   out_h(i)      = Wv_h (sum_j p_h(i, j) c(j))
// so attention runs over the cached rows themselves, as one shared key/value head of size R + dr whose
// values are the first R numbers of the key row; Wk is applied to the query before and Wv to the
// result after. Kernels here:
//   latent_prep       the two RMS norms behind the first product, rotation of kr, the cache write
//   latent_query      q -> [Wk_h^T qn_h | rot(qr_h)] per head
//   heads_product     out[t, h, :] = W_h a[t, h, :], optionally times sigmoid(gate[t, h, :])
//   latent_attention  softmax attention of every token over rows lo..pos of its request's pages
//   sigmoid_gate      x *= sigmoid(gate)
#include "common.cuh"

#include <cfloat>
#include <cmath>

namespace {

__device__ __forceinline__ float sum_parts(const float* __restrict__ parts, int n_parts, size_t pstride, size_t i) {
  float x = 0.f;
  for (int p0 = 0; p0 < n_parts; p0 += 4) {  // four parts' loads in flight, added in index order
    float v[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) v[k] = p0 + k < n_parts ? parts[(size_t)(p0 + k) * pstride + i] : 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) x += v[k];
  }
  return x;
}

// ------------------------------------------------------------------------------------ prep
// One block per token. parts [n_parts, tokens, width] float32: the product of the mixer's input with
// [Wdq; Wdkv; ...] as partial sums. Columns q_off .. q_off+Rq are the query latent, kv_off .. kv_off+R+dr
// the key/value latent followed by the part to rotate.
template <typename T>
__global__ void latent_prep_kernel(const float* __restrict__ parts, int n_parts, size_t pstride, int width, int q_off, int Rq,
                                   int kv_off, int R, int dr, int rot_dims, const float* __restrict__ wq, const float* __restrict__ wkv,
                                   float eps, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                   const int* __restrict__ positions, const int* __restrict__ token_seq,
                                   const int* __restrict__ block_table, int max_blocks, T* __restrict__ cq, long long ld_cq,
                                   T* __restrict__ cache, int page_size) {
  extern __shared__ float row[];  // Rq + R + dr
  __shared__ float red[33];
  dep_launch();
  dep_wait();
  const int tok = blockIdx.x;
  const size_t base = (size_t)tok * width;
  float ssq = 0.f, ssk = 0.f;
  for (int i = threadIdx.x; i < Rq; i += blockDim.x) {
    const float x = sum_parts(parts, n_parts, pstride, base + q_off + i);
    row[i] = x;
    ssq += x * x;
  }
  for (int i = threadIdx.x; i < R + dr; i += blockDim.x) {
    const float x = sum_parts(parts, n_parts, pstride, base + kv_off + i);
    row[Rq + i] = x;
    if (i < R) ssk += x * x;
  }
  ssq = block_sum(ssq, red);
  ssk = block_sum(ssk, red);
  const float iq = 1.0f / sqrtf(ssq / (float)Rq + eps), ik = 1.0f / sqrtf(ssk / (float)R + eps);
  T* q_out = cq + (size_t)tok * ld_cq;
  for (int i = threadIdx.x; i < Rq; i += blockDim.x) q_out[i] = from_f32<T>(row[i] * iq * wq[i]);
  if (cache == nullptr) return;
  const int pos = positions[tok];
  const int page = block_table[(size_t)token_seq[tok] * max_blocks + pos / page_size];
  T* dst = cache + ((size_t)page * page_size + (size_t)(pos % page_size)) * (size_t)(R + dr);
  for (int i = threadIdx.x; i < R; i += blockDim.x) dst[i] = from_f32<T>(row[Rq + i] * ik * wkv[i]);
  const int half = rot_dims / 2;
  const float* kr = row + Rq + R;
  for (int i = threadIdx.x; i < dr; i += blockDim.x) {
    float v = kr[i];
    if (i < half) {
      const float c = cos_t[(size_t)pos * half + i], s = sin_t[(size_t)pos * half + i];
      v = kr[i] * c - kr[i + half] * s;
    } else if (i < rot_dims) {
      const float c = cos_t[(size_t)pos * half + i - half], s = sin_t[(size_t)pos * half + i - half];
      v = kr[i] * c + kr[i - half] * s;
    }
    dst[R + i] = from_f32<T>(v);
  }
}

// ------------------------------------------------------------------------------------ per-head products
constexpr int HP_WARPS = 4, HP_TOKENS = 8;

__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8(const bf16* p, float (&v)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}

// One warp owns one output column n of one head for HP_TOKENS tokens: lanes stride over k (the weight
// row is read once, coalesced; eight numbers a lane a step where rows are 16-byte aligned, else one), then a
// shuffle tree; the order of additions depends on K and the alignment alone, never on the batch.
template <typename T>
__device__ __forceinline__ void warp_dots(const T* __restrict__ a, long long lda, const T* __restrict__ wrow, int K, int t0, int T_,
                                          float (&acc)[HP_TOKENS], bool vec) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int i = 0; i < HP_TOKENS; ++i) acc[i] = 0.f;
  if (vec) {
    for (int k = lane * 8; k < K; k += 256) {
      float wv[8];
      load8(wrow + k, wv);
#pragma unroll
      for (int i = 0; i < HP_TOKENS; ++i) {
        if (t0 + i < T_) {
          float av[8];
          load8(a + (size_t)(t0 + i) * lda + k, av);
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[i] = fmaf(av[e], wv[e], acc[i]);
        }
      }
    }
  } else {
    for (int k = lane; k < K; k += 32) {
      const float wv = to_f32(wrow[k]);
#pragma unroll
      for (int i = 0; i < HP_TOKENS; ++i)
        if (t0 + i < T_) acc[i] = fmaf(to_f32(a[(size_t)(t0 + i) * lda + k]), wv, acc[i]);
    }
  }
#pragma unroll
  for (int i = 0; i < HP_TOKENS; ++i) acc[i] = warp_sum(acc[i]);
}

// Whether rows of K numbers at these addresses and strides (in elements) can be read 16 bytes at a time.
template <typename T>
__device__ __forceinline__ bool rows_vectorizable(const T* a, long long lda, long long lda_h, const T* w, long long ldw, int K) {
  constexpr int per = 16 / sizeof(T);
  return K % 8 == 0 && (reinterpret_cast<uintptr_t>(a) & 15u) == 0 && (reinterpret_cast<uintptr_t>(w) & 15u) == 0 && lda % per == 0 &&
         lda_h % per == 0 && ldw % per == 0;
}

// out[t, h*ldo_h + n] = (sum_k a[t, h*lda_h + k] * w[(h*N + n), k]) (* sigmoid(sum_p gate[p][t][g_off + h*N + n]))
template <typename T>
__global__ void __launch_bounds__(HP_WARPS * 32)
    heads_product_kernel(const T* __restrict__ a, long long lda, long long lda_h, const T* __restrict__ w, long long ldw,
                         T* __restrict__ out, long long ldo, long long ldo_h, int T_, int N, int K,
                         const float* __restrict__ gate, int n_parts, size_t pstride, int gwidth, int g_off) {
  dep_launch();
  dep_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * HP_WARPS + warp, h = blockIdx.y, t0 = blockIdx.z * HP_TOKENS;
  if (n >= N) return;
  float acc[HP_TOKENS];
  warp_dots<T>(a + (size_t)h * lda_h, lda, w + ((size_t)h * N + n) * ldw, K, t0, T_, acc, rows_vectorizable(a, lda, lda_h, w, ldw, K));
  if (lane < HP_TOKENS && t0 + lane < T_) {
    float v = 0.f;
#pragma unroll
    for (int i = 0; i < HP_TOKENS; ++i)
      if (i == lane) v = acc[i];
    if (gate) {
      const float g = sum_parts(gate, n_parts, pstride, (size_t)(t0 + lane) * gwidth + g_off + (size_t)h * N + n);
      v *= 1.0f / (1.0f + expf(-g));
    }
    out[(size_t)(t0 + lane) * ldo + (size_t)h * ldo_h + n] = from_f32<T>(v);
  }
}

// q [tokens, H * (dn + dr)] -> ql [tokens, H, R + dr]: the first R numbers of a head are Wk_h^T qn_h
// (wkt [H, R, dn]: the head's key map, transposed), unless `absorb` is 0 (then somebody else writes
// them); the last dr are qr_h, its first rot_dims numbers rotated by the token's position.
template <typename T>
__global__ void __launch_bounds__(HP_WARPS * 32)
    latent_query_kernel(const T* __restrict__ q, long long ldq, const T* __restrict__ wkt, T* __restrict__ ql, int T_, int H,
                        int dn, int dr, int R, int rot_dims, int absorb, const float* __restrict__ cos_t,
                        const float* __restrict__ sin_t, const int* __restrict__ positions) {
  dep_launch();
  dep_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y, t0 = blockIdx.z * HP_TOKENS;
  const int n = blockIdx.x * HP_WARPS + warp + (absorb ? 0 : R);
  const size_t ldl = (size_t)H * (R + dr);
  if (n < R) {
    float acc[HP_TOKENS];
    warp_dots<T>(q + (size_t)h * (dn + dr), ldq, wkt + ((size_t)h * R + n) * dn, dn, t0, T_, acc,
                 rows_vectorizable(q, ldq, (long long)(dn + dr), wkt, (long long)dn, dn));
    if (lane < HP_TOKENS && t0 + lane < T_) {
      float v = 0.f;
#pragma unroll
      for (int i = 0; i < HP_TOKENS; ++i)
        if (i == lane) v = acc[i];
      ql[(size_t)(t0 + lane) * ldl + (size_t)h * (R + dr) + n] = from_f32<T>(v);
    }
    return;
  }
  const int j = n - R;
  if (j >= dr || lane >= HP_TOKENS || t0 + lane >= T_) return;
  const int t = t0 + lane, half = rot_dims / 2;
  const T* qr = q + (size_t)t * ldq + (size_t)h * (dn + dr) + dn;
  const int pos = positions[t];
  float v = to_f32(qr[j]);
  if (j < half) {
    v = v * cos_t[(size_t)pos * half + j] - to_f32(qr[j + half]) * sin_t[(size_t)pos * half + j];
  } else if (j < rot_dims) {
    v = v * cos_t[(size_t)pos * half + j - half] + to_f32(qr[j - half]) * sin_t[(size_t)pos * half + j - half];
  }
  ql[(size_t)t * ldl + (size_t)h * (R + dr) + R + j] = from_f32<T>(v);
}

// The rotated part alone (the unrotated part's map runs elsewhere): a thread a number.
template <typename T>
__global__ void latent_query_rotate_kernel(const T* __restrict__ q, long long ldq, T* __restrict__ ql, int H, int dn, int dr, int R,
                                           int rot_dims, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                           const int* __restrict__ positions, size_t total) {
  dep_launch();
  dep_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int j = (int)(i % dr);
  const size_t th = i / dr;
  const int h = (int)(th % H);
  const size_t t = th / H;
  const int half = rot_dims / 2;
  const T* qr = q + t * ldq + (size_t)h * (dn + dr) + dn;
  float v = to_f32(qr[j]);
  if (j < rot_dims) {
    const int pos = positions[t];
    if (j < half) v = v * cos_t[(size_t)pos * half + j] - to_f32(qr[j + half]) * sin_t[(size_t)pos * half + j];
    else v = v * cos_t[(size_t)pos * half + j - half] + to_f32(qr[j - half]) * sin_t[(size_t)pos * half + j - half];
  }
  ql[(t * H + h) * (size_t)(R + dr) + R + j] = from_f32<T>(v);
}

// ------------------------------------------------------------------------------------ attention
constexpr int LA_WARPS = 4;

// One warp owns one (token, head). Keys in chunks of 32 aligned to absolute positions with a running
// (max, sum): the chunking depends only on the token's position, so its result does not depend on how
// the request was cut into steps, on the rest of the batch or on page numbers. NV = ceil(R / 32).
template <typename T, int NV>
__global__ void __launch_bounds__(LA_WARPS * 32)
    latent_attention_simt_kernel(const T* __restrict__ ql, const T* __restrict__ cache, const int* __restrict__ positions,
                                 const int* __restrict__ token_seq, const int* __restrict__ block_table, int max_blocks,
                                 T* __restrict__ out, int n_tokens, int H, int R, int dr, int page_size, float scale, int window) {
  extern __shared__ float q_s[];  // LA_WARPS x (R + dr)
  dep_launch();
  dep_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * LA_WARPS + warp;
  if (item >= (long long)n_tokens * H) return;
  const int tok = (int)(item / H), head = (int)(item - (long long)tok * H);
  const int Dk = R + dr;
  const int pos = positions[tok];
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int* table = block_table + (size_t)token_seq[tok] * max_blocks;
  float* qs = q_s + (size_t)warp * Dk;
  const T* qv = ql + ((size_t)tok * H + head) * Dk;
  for (int d = lane; d < Dk; d += 32) qs[d] = to_f32(qv[d]);
  __syncwarp();

  float acc[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) acc[i] = 0.f;
  float m = -INFINITY, l = 0.f;
  for (int c = lo / 32; c <= pos / 32; ++c) {
    const int t = c * 32 + lane;
    const bool valid = (t >= lo) && (t <= pos);
    float s = -INFINITY;
    size_t off = 0;
    if (valid) {
      off = ((size_t)table[t / page_size] * page_size + (size_t)(t % page_size)) * Dk;
      const T* kr = cache + off;
      float dot = 0.f;
      for (int d = 0; d < Dk; ++d) dot = fmaf(qs[d], to_f32(kr[d]), dot);
      s = dot * scale;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float alpha = (m == -INFINITY) ? 0.f : expf(m - m_new);
    const float p = valid ? expf(s - m_new) : 0.f;
    l = l * alpha + warp_sum(p);
#pragma unroll
    for (int i = 0; i < NV; ++i) acc[i] *= alpha;
    const int j_end = min(32, pos - c * 32 + 1), j_begin = max(0, lo - c * 32);
    for (int j = j_begin; j < j_end; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const size_t off_j = __shfl_sync(0xffffffffu, (unsigned long long)off, j);
      const T* vr = cache + off_j;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int d = lane + 32 * i;
        if (d < R) acc[i] = fmaf(pj, to_f32(vr[d]), acc[i]);
      }
    }
    m = m_new;
  }
  const float inv = 1.0f / l;
  T* o = out + ((size_t)tok * H + head) * R;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int d = lane + 32 * i;
    if (d < R) o[d] = from_f32<T>(acc[i] * inv);
  }
}

template <typename T>
__global__ void sigmoid_gate_kernel(T* __restrict__ x, long long ldx, const float* __restrict__ gate, int n_parts, size_t pstride,
                                    int gwidth, int g_off, int cols, size_t total) {
  dep_launch();
  dep_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t r = i / cols;
  const int c = (int)(i - r * cols);
  const float g = sum_parts(gate, n_parts, pstride, r * gwidth + g_off + c);
  T* p = x + r * ldx + c;
  *p = from_f32<T>(to_f32(*p) / (1.0f + expf(-g)));
}

}  // namespace

extern "C" int llm_latent_prep(const float* parts, int n_parts, long long pstride, int width, int q_off, int Rq, int kv_off, int R,
                               int dr, int rot_dims, const float* wq, const float* wkv, float eps, const float* cos_t,
                               const float* sin_t, const int* positions, const int* token_seq, const int* block_table,
                               int max_blocks, void* cq, long long ld_cq, void* cache, int page_size, int dtype, int n_tokens,
                               cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(n_tokens > 0 && n_parts >= 1 && Rq > 0 && R > 0 && dr >= 0, "latent_prep: bad sizes");
  LLM_REQUIRE(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= dr, "latent_prep: %d rotated dimensions do not fit a part of %d", rot_dims, dr);
  LLM_REQUIRE(q_off >= 0 && kv_off >= 0 && q_off + Rq <= width && kv_off + R + dr <= width, "latent_prep: columns outside the product");
  LLM_REQUIRE(rot_dims == 0 || (cos_t && sin_t), "latent_prep: rotation tables missing");
  const size_t smem = (size_t)(Rq + R + dr) * sizeof(float);
  LLM_REQUIRE(smem <= 48 * 1024, "latent_prep: latent sizes %d + %d + %d exceed one block's shared memory", Rq, R, dr);
  if (dtype == LLM_F32)
    launch_kernel(latent_prep_kernel<float>, n_tokens, 256, smem, stream, parts, n_parts, (size_t)pstride, width, q_off, Rq, kv_off, R, dr,
                  rot_dims, wq, wkv, eps, cos_t, sin_t, positions, token_seq, block_table, max_blocks, (float*)cq, ld_cq, (float*)cache, page_size);
  else if (dtype == LLM_BF16)
    launch_kernel(latent_prep_kernel<bf16>, n_tokens, 256, smem, stream, parts, n_parts, (size_t)pstride, width, q_off, Rq, kv_off, R, dr,
                  rot_dims, wq, wkv, eps, cos_t, sin_t, positions, token_seq, block_table, max_blocks, (bf16*)cq, ld_cq, (bf16*)cache, page_size);
  else
    LLM_REQUIRE(false, "latent_prep: unknown dtype %d", dtype);
  LLM_CHECK_LAUNCH("latent_prep");
  return LLM_OK;
}

extern "C" int llm_heads_product(const void* a, long long lda, long long lda_h, const void* w, long long ldw, void* out, long long ldo,
                                 long long ldo_h, int n_tokens, int H, int N, int K, const float* gate, int n_parts, long long pstride,
                                 int gwidth, int g_off, int dtype, cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(n_tokens > 0 && H > 0 && N > 0 && K > 0 && H <= 65535, "heads_product: bad sizes");
  LLM_REQUIRE(ceil_div(n_tokens, HP_TOKENS) <= 65535, "heads_product: %d tokens are too many for one launch", n_tokens);
  dim3 grid(ceil_div(N, HP_WARPS), H, ceil_div(n_tokens, HP_TOKENS));
  if (dtype == LLM_F32)
    launch_kernel(heads_product_kernel<float>, grid, HP_WARPS * 32, 0, stream, (const float*)a, lda, lda_h, (const float*)w, ldw, (float*)out,
                  ldo, ldo_h, n_tokens, N, K, gate, n_parts, (size_t)pstride, gwidth, g_off);
  else if (dtype == LLM_BF16)
    launch_kernel(heads_product_kernel<bf16>, grid, HP_WARPS * 32, 0, stream, (const bf16*)a, lda, lda_h, (const bf16*)w, ldw, (bf16*)out,
                  ldo, ldo_h, n_tokens, N, K, gate, n_parts, (size_t)pstride, gwidth, g_off);
  else
    LLM_REQUIRE(false, "heads_product: unknown dtype %d", dtype);
  LLM_CHECK_LAUNCH("heads_product");
  return LLM_OK;
}

extern "C" int llm_latent_query(const void* q, long long ldq, const void* wkt, void* ql, int n_tokens, int H, int dn, int dr, int R,
                                int rot_dims, int absorb, const float* cos_t, const float* sin_t, const int* positions, int dtype,
                                cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(n_tokens > 0 && H > 0 && dn > 0 && dr >= 0 && R > 0 && H <= 65535, "latent_query: bad sizes");
  LLM_REQUIRE(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= dr, "latent_query: %d rotated dimensions do not fit a part of %d", rot_dims, dr);
  LLM_REQUIRE(ceil_div(n_tokens, HP_TOKENS) <= 65535, "latent_query: %d tokens are too many for one launch", n_tokens);
  const int cols = (absorb ? R : 0) + dr;
  if (cols == 0) return LLM_OK;
  if (!absorb) {
    const size_t total = (size_t)n_tokens * H * dr;
    const int blocks = ceil_div((long long)total, 256);
    if (dtype == LLM_F32)
      launch_kernel(latent_query_rotate_kernel<float>, blocks, 256, 0, stream, (const float*)q, ldq, (float*)ql, H, dn, dr, R, rot_dims, cos_t,
                    sin_t, positions, total);
    else if (dtype == LLM_BF16)
      launch_kernel(latent_query_rotate_kernel<bf16>, blocks, 256, 0, stream, (const bf16*)q, ldq, (bf16*)ql, H, dn, dr, R, rot_dims, cos_t,
                    sin_t, positions, total);
    else
      LLM_REQUIRE(false, "latent_query: unknown dtype %d", dtype);
    LLM_CHECK_LAUNCH("latent_query_rotate");
    return LLM_OK;
  }
  dim3 grid(ceil_div(cols, HP_WARPS), H, ceil_div(n_tokens, HP_TOKENS));
  if (dtype == LLM_F32)
    launch_kernel(latent_query_kernel<float>, grid, HP_WARPS * 32, 0, stream, (const float*)q, ldq, (const float*)wkt, (float*)ql, n_tokens, H,
                  dn, dr, R, rot_dims, absorb, cos_t, sin_t, positions);
  else if (dtype == LLM_BF16)
    launch_kernel(latent_query_kernel<bf16>, grid, HP_WARPS * 32, 0, stream, (const bf16*)q, ldq, (const bf16*)wkt, (bf16*)ql, n_tokens, H,
                  dn, dr, R, rot_dims, absorb, cos_t, sin_t, positions);
  else
    LLM_REQUIRE(false, "latent_query: unknown dtype %d", dtype);
  LLM_CHECK_LAUNCH("latent_query");
  return LLM_OK;
}

extern "C" int llm_latent_attention_simt(const void* ql, const void* cache, int dtype, const int* positions, const int* token_seq,
                                         const int* block_table, int max_blocks, void* out, int n_tokens, int H, int R, int dr,
                                         int page_size, float scale, int window, cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(n_tokens > 0 && H > 0 && R > 0 && dr >= 0, "latent_attention: bad sizes");
  LLM_REQUIRE(R <= 1024, "latent_attention: a latent of %d numbers is more than the CUDA-core kernel keeps (1024)", R);
  LLM_REQUIRE(page_size > 0 && max_blocks > 0 && window >= 0, "latent_attention: bad page_size/max_blocks/window");
  const size_t smem = (size_t)LA_WARPS * (R + dr) * sizeof(float);
  LLM_REQUIRE(smem <= 48 * 1024, "latent_attention: rows of %d numbers exceed one block's shared memory", R + dr);
  const int grid = ceil_div((long long)n_tokens * H, LA_WARPS);
#define LLM_LA_CASE(T, NV)                                                                                                        \
  launch_kernel(latent_attention_simt_kernel<T, NV>, grid, LA_WARPS * 32, smem, stream, (const T*)ql, (const T*)cache, positions, \
                token_seq, block_table, max_blocks, (T*)out, n_tokens, H, R, dr, page_size, scale, window)
#define LLM_LA_SIZES(T)              \
  if (R <= 64) LLM_LA_CASE(T, 2);    \
  else if (R <= 128) LLM_LA_CASE(T, 4); \
  else if (R <= 256) LLM_LA_CASE(T, 8); \
  else if (R <= 512) LLM_LA_CASE(T, 16); \
  else LLM_LA_CASE(T, 32)
  if (dtype == LLM_F32) {
    LLM_LA_SIZES(float);
  } else if (dtype == LLM_BF16) {
    LLM_LA_SIZES(bf16);
  } else {
    LLM_REQUIRE(false, "latent_attention: unknown dtype %d", dtype);
  }
#undef LLM_LA_SIZES
#undef LLM_LA_CASE
  LLM_CHECK_LAUNCH("latent_attention_simt");
  return LLM_OK;
}

extern "C" int llm_sigmoid_gate(void* x, long long ldx, const float* gate, int n_parts, long long pstride, int gwidth, int g_off,
                                int n_rows, int cols, int dtype, cudaStream_t stream) {
  if (n_rows == 0 || cols == 0) return LLM_OK;
  LLM_REQUIRE(n_rows > 0 && cols > 0 && n_parts >= 1 && g_off >= 0 && g_off + cols <= gwidth, "sigmoid_gate: bad sizes");
  const size_t total = (size_t)n_rows * cols;
  const int blocks = ceil_div((long long)total, 256);
  if (dtype == LLM_F32)
    launch_kernel(sigmoid_gate_kernel<float>, blocks, 256, 0, stream, (float*)x, ldx, gate, n_parts, (size_t)pstride, gwidth, g_off, cols, total);
  else if (dtype == LLM_BF16)
    launch_kernel(sigmoid_gate_kernel<bf16>, blocks, 256, 0, stream, (bf16*)x, ldx, gate, n_parts, (size_t)pstride, gwidth, g_off, cols, total);
  else
    LLM_REQUIRE(false, "sigmoid_gate: unknown dtype %d", dtype);
  LLM_CHECK_LAUNCH("sigmoid_gate");
  return LLM_OK;
}
