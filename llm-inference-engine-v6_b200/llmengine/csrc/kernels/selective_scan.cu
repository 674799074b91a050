// A recurrent mixer with input-dependent decay ("selective scan") over the step's flat ragged batch, float32 arithmetic.
// Per request the state lives in its slot: the last K - 1 inputs of the causal convolution [slots, K - 1, C] and the
// recurrent state [slots, C, N], both float32, zero when the request starts.
//
//   conv        xc[t, c] = silu(bias[c] + sum_j w[c, j] * x[t - (K - 1) + j, c]); inputs before the step's portion come
//               from the slot, inputs before the sequence are zero (the slot starts at zero)
//   conv_state  afterwards the slot holds the last K - 1 inputs again
//   dt          dt[t, c] = softplus(bias[c] + sum_r Wdt[c, r] * low[t, r])
//   scan        S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n;  y_c = sum_n S[c, n] C_n + D_c x_c;  out = y * silu(z)
//               with A = -exp(A_log); token after token of a request, the request's state read from and written to its slot
//
// x and z are columns of a product given as float32 partial sums [parts, tokens, width] (added in index order); low, B and C
// are columns of a float32 product [tokens, ld]. A token's result depends on the tokens before it in its request alone.
#include "common.cuh"

#include <cmath>

namespace {

__device__ __forceinline__ float parts_sum(const float* __restrict__ p, int n_parts, size_t pstride, size_t i) {
  float s = p[i];
  for (int k = 1; k < n_parts; ++k) s += p[(size_t)k * pstride + i];
  return s;
}

__device__ __forceinline__ float silu_f(float v) { return v / (1.0f + expf(-v)); }

constexpr int MAX_TAPS = 16;

template <typename T>
__global__ void conv_silu_kernel(const float* __restrict__ parts, int n_parts, size_t pstride, int width, int x_off, int C, int K,
                                 const T* __restrict__ w, const float* __restrict__ bias, const float* __restrict__ conv_state,
                                 const int* __restrict__ token_seq, const int* __restrict__ seq_qoff, const int* __restrict__ seq_slot,
                                 T* __restrict__ out, size_t total) {
  dep_launch();
  dep_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int tok = (int)(i / C), c = (int)(i - (size_t)tok * C);
  const int seq = token_seq[tok];
  const int first = seq_qoff[seq];
  const float* st = conv_state + (size_t)seq_slot[seq] * (K - 1) * C;
  float acc = bias ? bias[c] : 0.f;
  for (int j = 0; j < K; ++j) {
    const int src = tok - (K - 1) + j;  // flat row of the tap's input, if it is part of this step
    float v;
    if (src >= first) v = parts_sum(parts, n_parts, pstride, (size_t)src * width + x_off + c);
    else v = st[(size_t)((K - 1) + (src - first)) * C + c];  // src - first in [-(K-1), -1]
    acc = fmaf(to_f32(w[(size_t)c * K + j]), v, acc);
  }
  out[i] = from_f32<T>(silu_f(acc));
}

__global__ void conv_state_kernel(const float* __restrict__ parts, int n_parts, size_t pstride, int width, int x_off, int C, int K,
                                  float* __restrict__ conv_state, const int* __restrict__ seq_qoff, const int* __restrict__ seq_ntok,
                                  const int* __restrict__ seq_slot, int n_seqs) {
  dep_launch();
  dep_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)n_seqs * C) return;
  const int seq = (int)(i / C), c = (int)(i - (size_t)seq * C);
  const int first = seq_qoff[seq], n = seq_ntok[seq];
  float* st = conv_state + (size_t)seq_slot[seq] * (K - 1) * C;
  float keep[MAX_TAPS];
#pragma unroll
  for (int k = 0; k < MAX_TAPS; ++k) {
    if (k < K - 1) {
      const int rel = n - (K - 1) + k;  // which of the step's tokens, or (negative) how far back in the old state
      keep[k] = rel >= 0 ? parts_sum(parts, n_parts, pstride, (size_t)(first + rel) * width + x_off + c) : st[(size_t)(k + n) * C + c];
    }
  }
#pragma unroll
  for (int k = 0; k < MAX_TAPS; ++k)
    if (k < K - 1) st[(size_t)k * C + c] = keep[k];
}

constexpr int DT_TOKENS = 32, DT_THREADS = 128;

// wt: the step-size map stored [R, C] (transposed when loaded), so that neighbouring channels read neighbouring words
template <typename T>
__global__ void __launch_bounds__(DT_THREADS)
    dt_softplus_kernel(const float* __restrict__ proj, long long ld, int R, const T* __restrict__ wt, const float* __restrict__ bias, int C,
                       float* __restrict__ dt, int n_tokens) {
  extern __shared__ float low[];  // DT_TOKENS rows of R
  dep_launch();
  dep_wait();
  const int t0 = blockIdx.y * DT_TOKENS;
  for (int i = threadIdx.x; i < DT_TOKENS * R; i += blockDim.x) {
    const int t = t0 + i / R;
    low[i] = t < n_tokens ? proj[(size_t)t * ld + (i % R)] : 0.f;
  }
  __syncthreads();
  const int c = blockIdx.x * DT_THREADS + threadIdx.x;
  if (c >= C) return;
  float acc[DT_TOKENS];
#pragma unroll
  for (int i = 0; i < DT_TOKENS; ++i) acc[i] = 0.f;
#pragma unroll 4
  for (int r = 0; r < R; ++r) {
    const float wv = to_f32(wt[(size_t)r * C + c]);
#pragma unroll
    for (int i = 0; i < DT_TOKENS; ++i) acc[i] = fmaf(wv, low[i * R + r], acc[i]);
  }
  const float b = bias ? bias[c] : 0.f;
#pragma unroll
  for (int i = 0; i < DT_TOKENS; ++i) {
    const int t = t0 + i;
    if (t < n_tokens) {
      const float z = acc[i] + b;
      dt[(size_t)t * C + c] = z > 20.0f ? z : log1pf(expf(z));
    }
  }
}

constexpr int SCAN_THREADS = 128;
constexpr int SCAN_CHUNK = 64;  // tokens of a piece when a long portion is cut into pieces that run side by side

// How many pieces the requests before `seq` have (every request's portion is cut on its own).
__device__ __forceinline__ int pieces_before(const int* __restrict__ seq_ntok, int seq, int piece) {
  int n = 0;
  for (int s = 0; s < seq; ++s) n += (seq_ntok[s] + piece - 1) / piece;
  return n;
}

// TPC threads share a channel, each with NS of its N state numbers (n = part * NS + i). A block walks tokens of one request:
// MODE 0  the whole portion, from the request's slot and back into it;
// MODE 1  piece blockIdx.y of the portion, from a state of zero: leaves the piece's end state and the sum of its step sizes
//         (the decay over the piece is exp(A * that sum)), no outputs;
// MODE 2  the same piece again, from the state that the carry kernel has put at the piece's start: writes the outputs.
template <typename T, int NS, int MODE>
__global__ void __launch_bounds__(SCAN_THREADS)
    selective_scan_kernel(const T* __restrict__ xc, const float* __restrict__ dt, const float* __restrict__ proj, long long ld, int b_off,
                          int c_off, const float* __restrict__ zparts, int n_parts, size_t pstride, int zwidth, int z_off,
                          const float* __restrict__ a_log, const float* __restrict__ dskip, float* __restrict__ state,
                          const int* __restrict__ seq_qoff, const int* __restrict__ seq_ntok, const int* __restrict__ seq_slot, int C, int N,
                          int tpc, T* __restrict__ out, float* __restrict__ piece_state, float* __restrict__ piece_sumdt) {
  dep_launch();
  dep_wait();
  const int seq = blockIdx.z;
  int first = seq_qoff[seq], n_tok = seq_ntok[seq];
  size_t piece = 0;
  if (MODE != 0) {
    first += blockIdx.y * SCAN_CHUNK;
    n_tok = min(SCAN_CHUNK, n_tok - (int)blockIdx.y * SCAN_CHUNK);
    if (n_tok <= 0) return;
    piece = (size_t)pieces_before(seq_ntok, seq, SCAN_CHUNK) + blockIdx.y;
  }
  const int per_block = SCAN_THREADS / tpc;
  const int c = blockIdx.x * per_block + threadIdx.x / tpc;
  const int part = threadIdx.x % tpc;
  const bool live = c < C;
  const int cc = live ? c : C - 1;  // threads past the last channel compute along (the shuffles need them) and write nothing
  float* st = MODE == 0 ? state + ((size_t)seq_slot[seq] * C + cc) * N : piece_state + (piece * C + cc) * N;
  float S[NS], A[NS];
#pragma unroll
  for (int i = 0; i < NS; ++i) {
    const int n = part * NS + i;
    S[i] = (n < N && MODE != 1) ? st[n] : 0.f;
    A[i] = n < N ? -expf(a_log[(size_t)cc * N + n]) : 0.f;
  }
  const float dsk = dskip ? dskip[cc] : 0.f;
  float sum_dt = 0.f;
  for (int j = 0; j < n_tok; ++j) {
    const size_t t = (size_t)(first + j);
    const float d = dt[t * C + cc];
    const float x = to_f32(xc[t * C + cc]);
    const float* pr = proj + t * ld;
    const float dx = d * x;
    float y = 0.f;
    sum_dt += d;
#pragma unroll
    for (int i = 0; i < NS; ++i) {
      const int n = part * NS + i;
      if (n < N) {
        // exp(dA) S + dt x B as S + ((exp(dA) - 1) S + dt x B): a decay close to 1 is not rounded to the grid of floats around
        // 1 first, an error of the same sign token after token that would grow along a sequence where dA is small
        S[i] += fmaf(expm1f(d * A[i]), S[i], dx * pr[b_off + n]);
        if (MODE != 1) y = fmaf(S[i], pr[c_off + n], y);
      }
    }
    if (MODE != 1) {
      for (int o = tpc >> 1; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
      if (part == 0 && live) {
        const float z = parts_sum(zparts, n_parts, pstride, t * zwidth + z_off + cc);
        out[t * C + cc] = from_f32<T>((y + dsk * x) * silu_f(z));
      }
    }
  }
  if (live && MODE != 2) {
#pragma unroll
    for (int i = 0; i < NS; ++i) {
      const int n = part * NS + i;
      if (n < N) st[n] = S[i];
    }
    if (MODE == 1 && part == 0) piece_sumdt[piece * C + cc] = sum_dt;
  }
}

// Between the two passes over the pieces: a thread a (request, channel, state number) carries the state from the request's slot
// through its pieces, S <- exp(A * sum of the piece's step sizes) S + (the piece's end state from zero), leaves at every piece
// the state at its START (in place of the piece's own end state), and puts the last state back into the slot.
__global__ void scan_carry_kernel(const float* __restrict__ a_log, float* __restrict__ state, float* __restrict__ piece_state,
                                  const float* __restrict__ piece_sumdt, const int* __restrict__ seq_ntok, const int* __restrict__ seq_slot,
                                  int C, int N, int n_seqs) {
  dep_launch();
  dep_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t per_seq = (size_t)C * N;
  if (i >= per_seq * n_seqs) return;
  const int seq = (int)(i / per_seq);
  const size_t cn = i - (size_t)seq * per_seq;
  const int c = (int)(cn / N);
  const int pieces = (seq_ntok[seq] + SCAN_CHUNK - 1) / SCAN_CHUNK;
  const size_t base = (size_t)pieces_before(seq_ntok, seq, SCAN_CHUNK);
  const float A = -expf(a_log[cn]);
  float* slot = state + (size_t)seq_slot[seq] * per_seq + cn;
  float S = *slot;
  for (int j = 0; j < pieces; ++j) {
    float* ps = piece_state + (base + j) * per_seq + cn;
    const float local = *ps, sd = piece_sumdt[(base + j) * C + c];
    *ps = S;
    S += fmaf(expm1f(A * sd), S, local);
  }
  *slot = S;
}

}  // namespace

extern "C" int llm_conv_silu(const float* parts, int n_parts, long long pstride, int width, int x_off, int C, int K, const void* w,
                             const float* bias, float* conv_state, const int* token_seq, const int* seq_qoff, const int* seq_ntok,
                             const int* seq_slot, void* out, int dtype, int n_tokens, int n_seqs, cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(n_tokens > 0 && n_seqs > 0 && n_parts >= 1 && C > 0 && K >= 1 && K <= MAX_TAPS, "conv_silu: bad sizes (taps %d, at most %d)", K, MAX_TAPS);
  LLM_REQUIRE(x_off >= 0 && x_off + C <= width, "conv_silu: columns outside the product");
  const size_t total = (size_t)n_tokens * C;
  if (dtype == LLM_F32)
    launch_kernel(conv_silu_kernel<float>, ceil_div((long long)total, 256), 256, 0, stream, parts, n_parts, (size_t)pstride, width, x_off, C, K,
                  (const float*)w, bias, (const float*)conv_state, token_seq, seq_qoff, seq_slot, (float*)out, total);
  else if (dtype == LLM_BF16)
    launch_kernel(conv_silu_kernel<bf16>, ceil_div((long long)total, 256), 256, 0, stream, parts, n_parts, (size_t)pstride, width, x_off, C, K,
                  (const bf16*)w, bias, (const float*)conv_state, token_seq, seq_qoff, seq_slot, (bf16*)out, total);
  else
    LLM_REQUIRE(false, "conv_silu: unknown dtype %d", dtype);
  LLM_CHECK_LAUNCH("conv_silu");
  if (K > 1) {
    launch_kernel(conv_state_kernel, ceil_div((long long)n_seqs * C, 256), 256, 0, stream, parts, n_parts, (size_t)pstride, width, x_off, C, K,
                  conv_state, seq_qoff, seq_ntok, seq_slot, n_seqs);
    LLM_CHECK_LAUNCH("conv_state");
  }
  return LLM_OK;
}

extern "C" int llm_dt_softplus(const float* proj, long long ld, int R, const void* wt, const float* bias, int C, float* dt, int dtype,
                               int n_tokens, cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(n_tokens > 0 && R > 0 && C > 0 && R <= ld, "dt_softplus: bad sizes");
  const size_t smem = (size_t)DT_TOKENS * R * sizeof(float);
  LLM_REQUIRE(smem <= 48 * 1024, "dt_softplus: a step-size rank of %d exceeds one block's shared memory", R);
  dim3 grid(ceil_div(C, DT_THREADS), ceil_div(n_tokens, DT_TOKENS));
  LLM_REQUIRE(grid.y <= 65535, "dt_softplus: too many tokens in one step (%d)", n_tokens);
  if (dtype == LLM_F32)
    launch_kernel(dt_softplus_kernel<float>, grid, DT_THREADS, smem, stream, proj, ld, R, (const float*)wt, bias, C, dt, n_tokens);
  else if (dtype == LLM_BF16)
    launch_kernel(dt_softplus_kernel<bf16>, grid, DT_THREADS, smem, stream, proj, ld, R, (const bf16*)wt, bias, C, dt, n_tokens);
  else
    LLM_REQUIRE(false, "dt_softplus: unknown dtype %d", dtype);
  LLM_CHECK_LAUNCH("dt_softplus");
  return LLM_OK;
}

extern "C" int llm_selective_scan_piece() { return SCAN_CHUNK; }

// pieces > 0: the portions are cut into pieces of llm_selective_scan_piece() tokens that run side by side (two passes and a carry
// between them); piece_state holds pieces * C * N floats and piece_sumdt pieces * C, pieces >= the sum over the requests of
// ceil(tokens / piece), max_new_tokens = the longest portion. pieces == 0: every portion is walked by one block a channel tile.
extern "C" int llm_selective_scan(const void* xc, const float* dt, const float* proj, long long ld, int b_off, int c_off,
                                  const float* zparts, int n_parts, long long pstride, int zwidth, int z_off, const float* a_log,
                                  const float* dskip, float* state, const int* seq_qoff, const int* seq_ntok, const int* seq_slot, int C,
                                  int N, void* out, int dtype, int n_seqs, int max_new_tokens, int pieces, float* piece_state,
                                  float* piece_sumdt, cudaStream_t stream) {
  if (n_seqs == 0) return LLM_OK;
  LLM_REQUIRE(n_seqs > 0 && n_seqs <= 65535 && C > 0 && N > 0 && N <= 256, "selective_scan: bad sizes (state %d, at most 256)", N);
  LLM_REQUIRE(b_off >= 0 && c_off >= 0 && b_off + N <= ld && c_off + N <= ld && z_off >= 0 && z_off + C <= zwidth, "selective_scan: columns outside the products");
  LLM_REQUIRE(pieces == 0 || (piece_state && piece_sumdt && max_new_tokens > 0), "selective_scan: pieces need their scratch");
  const int ns = N <= 128 ? 4 : 8;
  int tpc = 1;
  while (tpc * ns < N) tpc <<= 1;  // a power of two up to 32
  const int per_seq_pieces = pieces ? ceil_div(max_new_tokens, SCAN_CHUNK) : 1;
  LLM_REQUIRE(per_seq_pieces <= 65535, "selective_scan: portion too long");
  dim3 grid(ceil_div(C, SCAN_THREADS / tpc), per_seq_pieces, n_seqs);
#define LLM_SCAN(T, NS, MODE)                                                                                                          \
  launch_kernel(selective_scan_kernel<T, NS, MODE>, grid, SCAN_THREADS, 0, stream, (const T*)xc, dt, proj, ld, b_off, c_off, zparts, n_parts, \
                (size_t)pstride, zwidth, z_off, a_log, dskip, state, seq_qoff, seq_ntok, seq_slot, C, N, tpc, (T*)out, piece_state, piece_sumdt)
#define LLM_SCAN_T(MODE)                                                                 \
  if (dtype == LLM_F32) { if (ns == 4) LLM_SCAN(float, 4, MODE); else LLM_SCAN(float, 8, MODE); } \
  else { if (ns == 4) LLM_SCAN(bf16, 4, MODE); else LLM_SCAN(bf16, 8, MODE); }
  LLM_REQUIRE(dtype == LLM_F32 || dtype == LLM_BF16, "selective_scan: unknown dtype %d", dtype);
  if (pieces == 0) {
    LLM_SCAN_T(0);
  } else {
    LLM_SCAN_T(1);
    LLM_CHECK_LAUNCH("selective_scan (pieces)");
    launch_kernel(scan_carry_kernel, ceil_div((long long)n_seqs * C * N, 256), 256, 0, stream, a_log, state, piece_state,
                  (const float*)piece_sumdt, seq_ntok, seq_slot, C, N, n_seqs);
    LLM_CHECK_LAUNCH("selective_scan (carry)");
    LLM_SCAN_T(2);
  }
#undef LLM_SCAN_T
#undef LLM_SCAN
  LLM_CHECK_LAUNCH("selective_scan");
  return LLM_OK;
}
