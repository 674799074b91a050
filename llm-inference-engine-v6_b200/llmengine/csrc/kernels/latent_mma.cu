// Latent attention on tensor cores (bfloat16 operands, float32 scores, statistics and accumulators), for
// prompt portions and decoded tokens alike.
//
// The cache holds one row [c | kr] of Dk = R + dr numbers per token; all heads read the same rows, as keys
// (all Dk numbers) and as values (the first R). A CTA owns one (request, tile of query tokens, tile of
// heads): its 32 rows are (token, head) pairs, so every row of a fetched key tile is used by all of them.
// Keys are walked in tiles of 64 aligned to absolute positions, fetched row by row through the block table
// with cp.async into double-buffered shared memory. Eight warps: two groups of 16 rows times four column
// warps. Per key tile, warp (g, c) first computes the scores of its 16 rows against keys 16c .. 16c+15 over
// all Dk numbers (m16n8k16), masks and scales them and leaves them in shared memory; after a barrier every
// warp reads the 64 scores of its rows, updates the running (max, sum) (the four column warps of a group do
// this alike, in the same order) and multiplies the probabilities (rounded to bfloat16) with its quarter of
// the value columns, R/4 accumulator columns a warp. Each row is masked by its own token's position (and
// window): the result for a token does not depend on what else is in the step.
// For decoding the key range is also cut into splits of a fixed number of keys (absolute boundaries); every
// split writes a normalised partial output with its (max, sum), and a second kernel merges them in index order.
#include "common.cuh"
#include "mma_common.cuh"

#include <cmath>

namespace {

constexpr int LM_CW = 4;  // column warps a group of rows
constexpr int lm_rows(int rgs) { return 16 * rgs; }
constexpr int lm_keys(int rgs) { return rgs == 4 ? 32 : 64; }

struct LatentParams {
  const bf16* ql;     // [tokens, H, Dk]
  const bf16* cache;  // [pages, page_size, Dk]
  const int* seq_start; const int* seq_ntok; const int* seq_qoff; const int* block_table;
  int max_blocks, H, gh, n_htiles, R, Dk, page_size, window;
  float scale;
  bf16* out;          // [tokens, H, R]
  float* part_o; float* part_ml; int split_keys, n_splits; long long n_tokens;
};

// DT: accumulator tiles of 16 columns a warp; R = 64 * DT. RGS: groups of 16 rows a CTA. 1: 16 rows, four warps (single
// tokens of up to 16 heads cut into splits; with splits of one key tile the CTA keeps one key buffer, 98 KB at 576
// numbers a row, and two CTAs share an SM). 2: 32 rows, key tiles of 64,
// eight warps (steps of single tokens and short portions, and rows whose length is no multiple of 32). 4: 64 rows, key
// tiles of 32, sixteen warps: the same shared memory holds twice the rows, so a fetched key row serves twice as many
// queries and twice the warps hide one another's waits (prompt portions).
template <int DT, bool SPLIT, int RGS>
__global__ void __launch_bounds__(RGS * 128) latent_attention_mma_kernel(const LatentParams p) {
  constexpr int LM_ROWS = 16 * RGS, LM_KEYS = RGS == 4 ? 32 : 64, LM_THREADS = RGS * 128, LM_SLD = LM_KEYS + 4;
  extern __shared__ __align__(16) uint8_t smem_raw[];
  const int Dk = p.Dk, LD = Dk + 8, CH = Dk / 8;  // padded row; 16-byte chunks of a row
  bf16* q_s = reinterpret_cast<bf16*>(smem_raw);            // [LM_ROWS][LD]
  bf16* k_s = q_s + LM_ROWS * LD;                           // [2][LM_KEYS][LD]
  const int buffers = (SPLIT && p.split_keys == LM_KEYS) ? 1 : 2;  // a split of one tile needs one buffer
  float* s_s = reinterpret_cast<float*>(k_s + buffers * LM_KEYS * LD);  // [LM_ROWS][LM_SLD]

  dep_launch();
  dep_wait();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rg = warp / LM_CW, cw = warp % LM_CW;
  const int seq = blockIdx.y;
  const int gh = min(p.H, LM_ROWS), tq_cap = LM_ROWS / gh;  // heads a tile, tokens a tile
  const int n_htiles = (p.H + gh - 1) / gh;
  const int htile = blockIdx.z % n_htiles, split = blockIdx.z / n_htiles;
  const int head0 = htile * gh;
  const int ntok = p.seq_ntok[seq];
  const int q0 = blockIdx.x * tq_cap;
  if (q0 >= ntok) return;
  const int n_tq = min(tq_cap, ntok - q0);
  const int tok_base = p.seq_qoff[seq] + q0;
  const int pos0 = p.seq_start[seq] + q0;
  const int pos_last = pos0 + n_tq - 1;
  int lo = (p.window > 0) ? max(0, pos0 - p.window + 1) : 0;
  int hi = pos_last;
  if (SPLIT) {
    lo = max(lo, split * p.split_keys);
    hi = min(hi, (split + 1) * p.split_keys - 1);
  }
  const int* table = p.block_table + (size_t)seq * p.max_blocks;
  auto row_valid = [&](int r) { return r < n_tq * gh && head0 + r % gh < p.H; };

  // ---- the query rows -> shared memory (padding rows are zeros). A warp copies whole rows, 16 bytes a lane, so
  // that rows and pages are worked out once a row and not once a copy (their sizes are no powers of two).
  for (int r = warp; r < LM_ROWS; r += LM_THREADS / 32) {
    const bool valid = row_valid(r);
    const bf16* src = valid ? p.ql + ((size_t)(tok_base + r / gh) * p.H + head0 + r % gh) * Dk : p.ql;
    // asynchronous copies (zeros for padding rows): all of a CTA's query rows are on their way at once, in the same
    // group as the first key tile
    for (int ch = lane; ch < CH; ch += 32) cp_async16(q_s + r * LD + ch * 8, src + (valid ? ch * 8 : 0), valid);
  }

  // A warp copies the tile's rows warp, warp + NW, ...; lane i first looks up where row i lies (one round of
  // block-table reads a tile, asked for one tile ahead of the copies that use them), then the copies follow.
  constexpr int NW = LM_THREADS / 32, RPW = LM_KEYS / NW;  // warps; rows of a tile a warp copies
  auto lookup = [&](int kt) -> long long {
    long long off = -1;  // -1: the row lies outside the keys this CTA reads (zeros are written instead)
    if (lane < RPW) {
      const int key = kt * LM_KEYS + warp + lane * NW;
      if (key >= lo && key <= hi) {
        const int pg = key / p.page_size;
        off = ((long long)table[pg] * p.page_size + (key - pg * p.page_size)) * Dk;
      }
    }
    return off;
  };
  auto load_tile = [&](int buf, long long my_off) {
    bf16* kd = k_s + (size_t)buf * LM_KEYS * LD;
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
      const long long off = __shfl_sync(0xffffffffu, my_off, i);
      const bool valid = off >= 0;
      bf16* dst = kd + (warp + i * NW) * LD;
      const bf16* src = p.cache + (valid ? off : 0);
      for (int ch = lane; ch < CH; ch += 32) cp_async16(dst + ch * 8, src + (valid ? ch * 8 : 0), valid);
    }
  };

  const int kt_first = lo / LM_KEYS, kt_last = hi / LM_KEYS;
  const bool any = hi >= lo;
  long long next_off = -1;
  if (any) {
    load_tile(0, lookup(kt_first));
    if (kt_first < kt_last) next_off = lookup(kt_first + 1);
  }
  cp_async_commit();

  const int row_a = rg * 16 + lane / 4, row_b = row_a + 8;  // the two rows this thread holds
  const int pos_a = row_valid(row_a) ? pos0 + row_a / gh : -1;  // -1: a padding row sees no key
  const int pos_b = row_valid(row_b) ? pos0 + row_b / gh : -1;
  const int lo_a = (p.window > 0) ? pos_a - p.window + 1 : 0, lo_b = (p.window > 0) ? pos_b - p.window + 1 : 0;

  float o_acc[2 * DT][4];
#pragma unroll
  for (int d = 0; d < 2 * DT; ++d) o_acc[d][0] = o_acc[d][1] = o_acc[d][2] = o_acc[d][3] = 0.f;
  float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
  const float sl2 = p.scale * 1.4426950408889634f;  // scores are kept in units of log2(e)

  if (any) {
    for (int kt = kt_first; kt <= kt_last; ++kt) {
      const int buf = (kt - kt_first) & 1;
      if (kt < kt_last) {
        load_tile(buf ^ 1, next_off);
        if (kt + 1 < kt_last) next_off = lookup(kt + 2);  // used an iteration from now
      }
      cp_async_commit();
      cp_async_wait<1>();
      __syncthreads();  // tile kt (and, the first time, the query rows) visible
      const bf16* kb = k_s + (size_t)buf * LM_KEYS * LD;

      // ---- scores of this warp's 16 rows against its share of the tile's keys, over all Dk numbers
      if (LM_KEYS == 64) {  // 16 keys a warp: two accumulator tiles
        float s[2][4];
        s[0][0] = s[0][1] = s[0][2] = s[0][3] = s[1][0] = s[1][1] = s[1][2] = s[1][3] = 0.f;
        const bf16* qrow = q_s + (rg * 16 + (lane % 16)) * LD + (lane / 16) * 8;
        const bf16* krow = kb + (cw * 16 + (lane % 8) + (lane / 16) * 8) * LD + ((lane / 8) % 2) * 8;
#pragma unroll 4
        for (int ks = 0; ks < Dk / 16; ++ks) {
          uint32_t a[4], b[4];
          ldmatrix_x4(a, qrow + ks * 16);
          ldmatrix_x4(b, krow + ks * 16);
          mma_bf16(s[0], a, b[0], b[1]);
          mma_bf16(s[1], a, b[2], b[3]);
        }
        const int col0 = cw * 16 + 2 * (lane % 4);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int col = col0 + j * 8 + e;
            const int key = kt * LM_KEYS + col;
            const bool in_split = key >= lo && key <= hi;
            const bool va = in_split && key <= pos_a && key >= lo_a;
            const bool vb = in_split && key <= pos_b && key >= lo_b;
            s_s[row_a * LM_SLD + col] = va ? s[j][e] * sl2 : -INFINITY;
            s_s[row_b * LM_SLD + col] = vb ? s[j][2 + e] * sl2 : -INFINITY;
          }
        }
      } else {  // 8 keys a warp: one ldmatrix brings the keys' numbers of two k-steps; even and odd steps sum apart
        float se[4] = {0.f, 0.f, 0.f, 0.f}, so[4] = {0.f, 0.f, 0.f, 0.f};
        const bf16* qrow = q_s + (rg * 16 + (lane % 16)) * LD + (lane / 16) * 8;
        const bf16* krow = kb + (cw * 8 + (lane % 8)) * LD + (lane / 8) * 8;
#pragma unroll 2
        for (int ks = 0; ks < Dk / 16; ks += 2) {
          uint32_t a0[4], a1[4], b[4];
          ldmatrix_x4(a0, qrow + ks * 16);
          ldmatrix_x4(a1, qrow + ks * 16 + 16);
          ldmatrix_x4(b, krow + ks * 16);
          mma_bf16(se, a0, b[0], b[1]);
          mma_bf16(so, a1, b[2], b[3]);
        }
        const int col0 = cw * 8 + 2 * (lane % 4);
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int col = col0 + e;
          const int key = kt * LM_KEYS + col;
          const bool in_split = key >= lo && key <= hi;
          const bool va = in_split && key <= pos_a && key >= lo_a;
          const bool vb = in_split && key <= pos_b && key >= lo_b;
          s_s[row_a * LM_SLD + col] = va ? (se[e] + so[e]) * sl2 : -INFINITY;
          s_s[row_b * LM_SLD + col] = vb ? (se[2 + e] + so[2 + e]) * sl2 : -INFINITY;
        }
      }
      __syncthreads();  // all scores of every row are there

      // ---- running softmax of rows a and b over the 64 keys (float32), then O += P V on this warp's columns
      float s2[LM_KEYS / 8][4];
      float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
      for (int j = 0; j < LM_KEYS / 8; ++j) {
        const float2 va = *reinterpret_cast<const float2*>(s_s + row_a * LM_SLD + j * 8 + 2 * (lane % 4));
        const float2 vb = *reinterpret_cast<const float2*>(s_s + row_b * LM_SLD + j * 8 + 2 * (lane % 4));
        s2[j][0] = va.x; s2[j][1] = va.y; s2[j][2] = vb.x; s2[j][3] = vb.y;
        mx_a = fmaxf(mx_a, fmaxf(va.x, va.y));
        mx_b = fmaxf(mx_b, fmaxf(vb.x, vb.y));
      }
      mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
      mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
      mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
      mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
      const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
      const float base_a = (mn_a == -INFINITY) ? 0.f : mn_a, base_b = (mn_b == -INFINITY) ? 0.f : mn_b;
      const float al_a = exp2f(m_a - base_a), al_b = exp2f(m_b - base_b);  // exp2(-inf) = 0 on the first tile
      float sum_a = 0.f, sum_b = 0.f;
#pragma unroll
      for (int j = 0; j < LM_KEYS / 8; ++j) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          s2[j][e] = exp2f(s2[j][e] - base_a);
          s2[j][2 + e] = exp2f(s2[j][2 + e] - base_b);
          sum_a += s2[j][e];
          sum_b += s2[j][2 + e];
        }
      }
      sum_a += __shfl_xor_sync(0xffffffffu, sum_a, 1);
      sum_a += __shfl_xor_sync(0xffffffffu, sum_a, 2);
      sum_b += __shfl_xor_sync(0xffffffffu, sum_b, 1);
      sum_b += __shfl_xor_sync(0xffffffffu, sum_b, 2);
      l_a = l_a * al_a + sum_a;
      l_b = l_b * al_b + sum_b;
      m_a = mn_a;
      m_b = mn_b;
#pragma unroll
      for (int d = 0; d < 2 * DT; ++d) {
        o_acc[d][0] *= al_a; o_acc[d][1] *= al_a;
        o_acc[d][2] *= al_b; o_acc[d][3] *= al_b;
      }
#pragma unroll
      for (int kk = 0; kk < LM_KEYS / 16; ++kk) {
        uint32_t pa[4];
        pa[0] = pack_bf16(s2[2 * kk][0], s2[2 * kk][1]);
        pa[1] = pack_bf16(s2[2 * kk][2], s2[2 * kk][3]);
        pa[2] = pack_bf16(s2[2 * kk + 1][0], s2[2 * kk + 1][1]);
        pa[3] = pack_bf16(s2[2 * kk + 1][2], s2[2 * kk + 1][3]);
        const bf16* vrow = kb + (kk * 16 + (lane % 8) + ((lane / 8) % 2) * 8) * LD + cw * DT * 16 + (lane / 16) * 8;
#pragma unroll
        for (int d2 = 0; d2 < DT; ++d2) {
          uint32_t b[4];
          ldmatrix_x4_trans(b, vrow + d2 * 16);
          mma_bf16(o_acc[2 * d2], pa, b[0], b[1]);
          mma_bf16(o_acc[2 * d2 + 1], pa, b[2], b[3]);
        }
      }
      __syncthreads();  // everyone is done with this buffer and with the scores before they are written again
    }
  }
  cp_async_wait<0>();

  // ---- write: rows a and b of this thread, columns 2*(lane%4)+{0,1} of every 8-wide tile of this warp's quarter
  const float inv_a = l_a > 0.f ? 1.f / l_a : 0.f, inv_b = l_b > 0.f ? 1.f / l_b : 0.f;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int row = half ? row_b : row_a;
    if (!row_valid(row)) continue;
    const int tok = tok_base + row / gh, head = head0 + row % gh;
    const float inv = half ? inv_b : inv_a;
    const int col0 = cw * DT * 16 + 2 * (lane % 4);
    if (!SPLIT) {
      bf16* dst = p.out + ((size_t)tok * p.H + head) * p.R + col0;
#pragma unroll
      for (int d = 0; d < 2 * DT; ++d)
        *reinterpret_cast<uint32_t*>(dst + d * 8) = pack_bf16(o_acc[d][2 * half] * inv, o_acc[d][2 * half + 1] * inv);
    } else {
      const size_t slot = ((size_t)split * p.n_tokens + tok) * p.H + head;
      float* dst = p.part_o + slot * p.R + col0;
#pragma unroll
      for (int d = 0; d < 2 * DT; ++d)
        *reinterpret_cast<float2*>(dst + d * 8) = make_float2(o_acc[d][2 * half] * inv, o_acc[d][2 * half + 1] * inv);
      if (cw == 0 && (lane % 4) == 0) {
        p.part_ml[slot * 2] = half ? m_b : m_a;  // log2 units; -inf when this split saw no key of the row
        p.part_ml[slot * 2 + 1] = half ? l_b : l_a;
      }
    }
  }
}

// Merges the splits of every (token, head) in index order: out = sum_s w_s o_s / sum_s w_s, w_s = l_s * 2^(m_s - max m).
// One block per (token, head): the weights are computed once into shared memory, then every thread owns columns.
constexpr int LC_THREADS = 256, LC_MAX_SPLITS = 128;
__global__ void __launch_bounds__(LC_THREADS)
    latent_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, int n_splits, long long n_tokens, int H,
                          int R, bf16* __restrict__ out) {
  __shared__ float w_s[LC_MAX_SPLITS];
  __shared__ float red[33];
  dep_launch();
  dep_wait();
  const size_t item = blockIdx.x;
  const size_t split_stride = (size_t)n_tokens * H;
  const int tid = threadIdx.x;
  float m = -INFINITY, l = 0.f;
  if (tid < n_splits) {
    m = part_ml[(item + tid * split_stride) * 2];
    l = part_ml[(item + tid * split_stride) * 2 + 1];
  }
  // block maximum (warp maxima through shared memory)
  float mx = warp_max(m);
  if ((tid & 31) == 0) red[tid >> 5] = mx;
  __syncthreads();
  mx = red[0];
#pragma unroll
  for (int i = 1; i < LC_THREADS / 32; ++i) mx = fmaxf(mx, red[i]);
  if (tid < LC_MAX_SPLITS) w_s[tid] = (tid < n_splits && m != -INFINITY) ? l * exp2f(m - mx) : 0.f;
  __syncthreads();
  float den = 0.f;
  for (int s = 0; s < n_splits; ++s) den += w_s[s];  // index order, the same in every thread
  const float inv = den > 0.f ? 1.f / den : 0.f;
  for (int d = tid; d < R; d += LC_THREADS) {
    float acc = 0.f;
    for (int s0 = 0; s0 < n_splits; s0 += 8) {  // eight loads in flight, added in index order
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = (s0 + u < n_splits && w_s[s0 + u] != 0.f) ? part_o[(item + (s0 + u) * split_stride) * R + d] : 0.f;
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (s0 + u < n_splits) acc = fmaf(w_s[s0 + u], v[u], acc);
    }
    out[item * R + d] = __float2bfloat16_rn(acc * inv);
  }
}

// buffers: 2, or 1 for CTAs that read a single key tile (splits of 64 keys): the second buffer is never touched then
size_t latent_smem(int Dk, int rgs = 2, int buffers = 2) {
  return (size_t)(lm_rows(rgs) + buffers * lm_keys(rgs)) * (Dk + 8) * sizeof(bf16) + (size_t)lm_rows(rgs) * (lm_keys(rgs) + 4) * sizeof(float);
}

template <int DT, bool SPLIT, int RGS>
int launch_latent_as(const LatentParams& p, dim3 grid, cudaStream_t stream) {
  const size_t smem = latent_smem(p.Dk, RGS, (SPLIT && p.split_keys == lm_keys(RGS)) ? 1 : 2);
  if (smem > 48 * 1024 && cudaFuncSetAttribute(latent_attention_mma_kernel<DT, SPLIT, RGS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    return 1;
  launch_kernel(latent_attention_mma_kernel<DT, SPLIT, RGS>, grid, RGS * 128, smem, stream, p);
  return 0;
}

template <int DT>
int launch_latent(const LatentParams& p, dim3 grid, bool split, bool wide, cudaStream_t stream) {
  // single tokens: 16 rows a CTA where the heads fit them (a smaller footprint: two CTAs an SM), else 32
  if (split) return p.gh <= 16 ? launch_latent_as<DT, true, 1>(p, grid, stream) : launch_latent_as<DT, true, 2>(p, grid, stream);
  return wide ? launch_latent_as<DT, false, 4>(p, grid, stream) : launch_latent_as<DT, false, 2>(p, grid, stream);
}

}  // namespace

// Whether the tensor-core kernel takes this geometry (else the caller uses the CUDA-core kernel): a latent of
// 64, 128, ... 512 numbers, a rotated part that is a multiple of 16, rows that fit shared memory.
extern "C" int llm_latent_attention_mma_supported(int H, int R, int dr) {
  return H > 0 && R >= 64 && R % 64 == 0 && R <= 512 && dr >= 0 && dr % 16 == 0 && latent_smem(R + dr) <= 220 * 1024;
}

extern "C" long long llm_latent_attention_scratch_floats(int n_tokens, int H, int R, int n_splits) {
  return (long long)n_splits * n_tokens * H * (R + 2);
}

// ql [tokens, H, R+dr] bf16; cache [pages, 1, page_size, R+dr] bf16; out [tokens, H, R] bf16. n_splits > 1 (steps of
// single tokens only): keys are cut every split_keys (a multiple of 64) positions; scratch holds
// llm_latent_attention_scratch_floats floats.
extern "C" int llm_latent_attention_mma(const void* ql, const void* cache, const int* seq_start, const int* seq_ntok,
                                        const int* seq_qoff, const int* block_table, int max_blocks, void* out, int n_seqs,
                                        int n_tokens, int max_new_tokens, int H, int R, int dr, int page_size, float scale, int window,
                                        int n_splits, int split_keys, float* scratch, cudaStream_t stream) {
  if (n_tokens == 0 || n_seqs == 0) return LLM_OK;
  LLM_REQUIRE(llm_latent_attention_mma_supported(H, R, dr), "latent_attention_mma: geometry not supported (heads=%d latent=%d rotated=%d)", H, R, dr);
  LLM_REQUIRE(page_size > 0 && max_blocks > 0 && window >= 0 && max_new_tokens > 0, "latent_attention_mma: bad sizes");
  LLM_REQUIRE((reinterpret_cast<uintptr_t>(ql) & 15u) == 0 && (reinterpret_cast<uintptr_t>(cache) & 15u) == 0,
              "latent_attention_mma: queries and cache must be 16-byte aligned");
  LLM_REQUIRE(n_splits <= LC_MAX_SPLITS, "latent_attention_mma: at most %d splits", LC_MAX_SPLITS);
  LLM_REQUIRE(n_splits >= 1 && (n_splits == 1 || (split_keys > 0 && split_keys % 64 == 0 && scratch != nullptr && max_new_tokens == 1)),
              "latent_attention_mma: splits need single tokens, split_keys %% 64 == 0 and scratch");
  LatentParams p;
  p.ql = (const bf16*)ql; p.cache = (const bf16*)cache; p.seq_start = seq_start; p.seq_ntok = seq_ntok; p.seq_qoff = seq_qoff;
  // the wide form (64 rows a CTA) for steps with portions of at least 64 rows, where rows are a multiple of 32 numbers
  const bool split = n_splits > 1;
  const bool wide = !split && (long long)max_new_tokens * H >= 64 && (R + dr) % 32 == 0 && latent_smem(R + dr, 4) <= 220 * 1024;
  const int rows = lm_rows(wide ? 4 : (split && H <= 16 ? 1 : 2));
  p.block_table = block_table; p.max_blocks = max_blocks; p.H = H; p.gh = H < rows ? H : rows;
  p.n_htiles = (H + p.gh - 1) / p.gh; p.R = R; p.Dk = R + dr; p.page_size = page_size; p.window = window; p.scale = scale;
  p.out = (bf16*)out; p.n_splits = n_splits; p.split_keys = split_keys; p.n_tokens = n_tokens;
  p.part_o = scratch; p.part_ml = scratch ? scratch + (size_t)n_splits * n_tokens * H * R : nullptr;
  const int tq_cap = rows / p.gh;
  LLM_REQUIRE((long long)n_seqs <= 65535 && (long long)p.n_htiles * n_splits <= 65535, "latent_attention_mma: batch too large for the grid");
  dim3 grid((max_new_tokens + tq_cap - 1) / tq_cap, n_seqs, p.n_htiles * n_splits);
  int rc = 0;
  switch (R / 64) {
    case 1: rc = launch_latent<1>(p, grid, split, wide, stream); break;
    case 2: rc = launch_latent<2>(p, grid, split, wide, stream); break;
    case 3: rc = launch_latent<3>(p, grid, split, wide, stream); break;
    case 4: rc = launch_latent<4>(p, grid, split, wide, stream); break;
    case 5: rc = launch_latent<5>(p, grid, split, wide, stream); break;
    case 6: rc = launch_latent<6>(p, grid, split, wide, stream); break;
    case 7: rc = launch_latent<7>(p, grid, split, wide, stream); break;
    default: rc = launch_latent<8>(p, grid, split, wide, stream); break;
  }
  LLM_REQUIRE(rc == 0, "latent_attention_mma: cannot raise the shared memory limit");
  if (split) {
    const long long items = (long long)n_tokens * H;
    launch_kernel(latent_combine_kernel, (int)items, LC_THREADS, 0, stream, (const float*)p.part_o, (const float*)p.part_ml, n_splits,
                  (long long)n_tokens, H, R, (bf16*)out);
  }
  LLM_CHECK_LAUNCH("latent_attention_mma");
  return LLM_OK;
}
