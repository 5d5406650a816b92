// Kernels for a decoder whose residual is several streams (hyper-connections), whose attention has a short causal
// convolution over time behind its projections, and whose recurrent mixer lets one gate decide what a state forgets
// and what it takes in.
//
//   stream_norm      the residual as S streams x_1 .. x_S of a token, [N][S][W] float32.  First the pending sublayer
//                    result y (up to four pending sums, each a [N, W] array or a K-split stack with a scale, times a
//                    layer scale [W]) joins them, all new streams from the old ones:
//                        x_t <- sum_s mix[s][t] x_s + out[t] y
//                    then the next sublayer's input u = sum_t in[t] x_t is formed and normed,
//                        out = u / sqrt(mean(u^2) + eps) * w,
//                    in one pass over the row.  On gathered rows (the final norm) the streams are left as they are.
//   short_conv       c_t = sum_j taps[:, j] u_(t - T + 1 + j) on every channel of a fused projection, the T - 1
//                    projected values before a portion's first token taken from the request's state (zeros at a
//                    sequence's start); short_conv_keep leaves the last T - 1 projected values there.
//   gated_scan       per head S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T, o_t = S_t^T q_t with q = silu(.) and
//                    f = lower + (1 - lower) sigmoid(. + bias), token by token with the state slice in registers; for long
//                    portions in three launches over runs of tokens (every run from a zero state and its decay, the
//                    runs' states carried in order, every run again from the state it starts from).
//   head_rms         every head of a row over its root mean square, times one weight of the head's size.
//
// Sums, norms, gates, decays and states are float32; a result is rounded once, when it is stored in the activation type.
#include <cooperative_groups.h>

#include "common.cuh"

namespace streams {
namespace cg = cooperative_groups;

constexpr int MAX_STREAMS = 8;
constexpr int MAX_TERMS = 4;

struct Term {
  const float* data;      // [partials][N][W]
  long long stride;       // elements between partials
  int partials;
  float scale;
};

struct StreamNormArgs {
  float* x;                  // [N][S][W]
  Term terms[MAX_TERMS];
  int num_terms;
  const float* mix;          // [S][S], (from, to), of the pending sublayer; null: nothing is pending
  const float* out_w;        // [S]
  const float* layer_scale;  // [W] or null
  const float* in_w;         // [S]; null: every stream counts once (the sum of the streams)
  const float* norm_w;       // [W]; null: no norm, `sum_out` alone
  float eps;
  void* out;                 // [rows][W] in the activation type, or null
  float* sum_out;            // [rows][W] float32 or null: u itself
  const int* rows;           // null: every row, streams rewritten; else row r of the outputs is token rows[r]
  int n, width, count;
  int split;                 // CTAs that share a row (a thread-block cluster along x): few rows are spread over the GPU
};

// MAXS: the most streams an instance holds in registers (1, 2, 4 or 8): fewer registers, more rows under way an SM
template <typename TO, int VEC, int MAXS>
__global__ void __launch_bounds__(256, MAXS <= 4 ? 3 : 2) stream_norm_kernel(const StreamNormArgs a) {
  extern __shared__ float stream_shared[];   // [width] u, then 33 floats for the block's sum
  __shared__ float mix[MAX_STREAMS * MAX_STREAMS], out_w[MAX_STREAMS], in_w[MAX_STREAMS];
  let_dependents_start();
  const int S = a.count;
  const bool pending = a.mix != nullptr;
  // parameters of the model: no kernel writes them, so they may be read before the wait
  for (int i = threadIdx.x; i < S * S; i += blockDim.x) mix[i] = pending ? a.mix[i] : 0.f;
  for (int i = threadIdx.x; i < S; i += blockDim.x) {
    out_w[i] = pending ? a.out_w[i] : 0.f;
    in_w[i] = a.in_w != nullptr ? a.in_w[i] : 1.f;
  }
  wait_for_previous();
  __syncthreads();
  float* u_row = stream_shared;
  float* scratch = stream_shared + a.width;
  const int groups = a.width / VEC;
  // A row's columns are dealt to the `split` CTAs of a cluster; their sums of squares meet through distributed shared
  // memory, added in the order of the ranks by every CTA alike.
  __shared__ float share;
  const int split = a.split, rank = split > 1 ? static_cast<int>(blockIdx.x % split) : 0;
  const int group_lo = static_cast<int>(static_cast<long long>(groups) * rank / split);
  const int group_hi = static_cast<int>(static_cast<long long>(groups) * (rank + 1) / split);
  for (int row = blockIdx.x / split; row < a.n; row += gridDim.x / split) {
    const int src = a.rows != nullptr ? a.rows[row] : row;
    float* x = a.x + static_cast<size_t>(src) * S * a.width;
    const size_t term_base = static_cast<size_t>(src) * a.width;
    float squares = 0.f;
    for (int group = group_lo + threadIdx.x; group < group_hi; group += blockDim.x) {
      const int col = group * VEC;
      float old[MAXS][VEC];
#pragma unroll
      for (int s = 0; s < MAXS; ++s) {
        if (s < S) {
          if constexpr (VEC == 4) load4<float>(x + static_cast<size_t>(s) * a.width + col, old[s]);
          else old[s][0] = x[static_cast<size_t>(s) * a.width + col];
        }
      }
      float y[VEC];
#pragma unroll
      for (int e = 0; e < VEC; ++e) y[e] = 0.f;
      if (pending) {
        for (int t = 0; t < a.num_terms; ++t) {
          const Term& term = a.terms[t];
          float part[VEC];
          if constexpr (VEC == 4) sum_partials4(term.data + term_base + col, term.stride, term.partials, part);
          else part[0] = sum_partials(term.data + term_base + col, term.stride, term.partials);
#pragma unroll
          for (int e = 0; e < VEC; ++e) y[e] = __fmaf_rn(term.scale, part[e], y[e]);
        }
        if (a.layer_scale != nullptr) {
#pragma unroll
          for (int e = 0; e < VEC; ++e) y[e] = __fmul_rn(y[e], a.layer_scale[col + e]);
        }
      }
      float u[VEC];
#pragma unroll
      for (int e = 0; e < VEC; ++e) u[e] = 0.f;
#pragma unroll
      for (int t = 0; t < MAXS; ++t) {
        if (t < S) {
          float fresh[VEC];
          if (pending) {
#pragma unroll
            for (int e = 0; e < VEC; ++e) fresh[e] = __fmul_rn(out_w[t], y[e]);
#pragma unroll
            for (int s = 0; s < MAXS; ++s)
              if (s < S) {
#pragma unroll
                for (int e = 0; e < VEC; ++e) fresh[e] = __fmaf_rn(mix[s * S + t], old[s][e], fresh[e]);
              }
            if (a.rows == nullptr) {
              if constexpr (VEC == 4) store4<float>(x + static_cast<size_t>(t) * a.width + col, fresh);
              else x[static_cast<size_t>(t) * a.width + col] = fresh[0];
            }
          } else {
#pragma unroll
            for (int e = 0; e < VEC; ++e) fresh[e] = old[t][e];
          }
#pragma unroll
          for (int e = 0; e < VEC; ++e) u[e] = __fmaf_rn(in_w[t], fresh[e], u[e]);
        }
      }
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        u_row[col + e] = u[e];
        squares = __fmaf_rn(u[e], u[e], squares);
      }
    }
    if (a.sum_out != nullptr) {
      __syncthreads();
      for (int col = group_lo * VEC + threadIdx.x; col < group_hi * VEC; col += blockDim.x)
        a.sum_out[static_cast<size_t>(row) * a.width + col] = u_row[col];
    }
    if (a.norm_w == nullptr || a.out == nullptr) {
      __syncthreads();
      continue;
    }
    float total = block_sum(squares, scratch);
    if (split > 1) {
      cg::cluster_group cluster = cg::this_cluster();
      if (threadIdx.x == 0) share = total;
      cluster.sync();
      total = 0.f;
      for (int other = 0; other < split; ++other) total += *cluster.map_shared_rank(&share, other);
      cluster.sync();   // every CTA has read every share before one of them is written again or its CTA leaves
    }
    const float r = rsqrtf(total / static_cast<float>(a.width) + a.eps);
    TO* out = static_cast<TO*>(a.out) + static_cast<size_t>(row) * a.width;
    for (int group = group_lo + threadIdx.x; group < group_hi; group += blockDim.x) {
      const int col = group * VEC;
      if constexpr (VEC == 4) {
        float w[4], v[4];
        load4<float>(a.norm_w + col, w);
#pragma unroll
        for (int e = 0; e < 4; ++e) v[e] = u_row[col + e] * r * w[e];
        store4<TO>(out + col, v);
      } else {
        out[col] = from_float<TO>(u_row[col] * r * a.norm_w[col]);
      }
    }
    __syncthreads();   // the row's buffer is free for the next row
  }
}

// ------------------------------------------------------------------------------------------------ short_conv
constexpr int MAX_TAPS = 32;

struct ConvArgs {
  const float* fused;     // [partials][N][total]; the first `channels` columns are convolved, the rest pass
  long long stride;
  int partials, total;
  const float* bias;      // [total] or null: part of the projected value
  const float* taps;      // [channels][T]
  float* state;           // [slots][T - 1][channels]: the last projected values, the newest last
  const int* q_start;     // [S + 1]
  const int* state_slot;  // [S]; -1: no state (zeros are read, nothing is kept)
  const int* seq_of_token;
  float* out;             // [N][total]
  int n, channels, taps_count, num_seqs, num_slots;
};

__device__ __forceinline__ float projected(const ConvArgs& a, int token, int c) {
  float v = sum_partials(a.fused + static_cast<size_t>(token) * a.total + c, a.stride, a.partials);
  if (a.bias != nullptr) v = __fadd_rn(v, a.bias[c]);
  return v;
}

__global__ void __launch_bounds__(256) short_conv_kernel(const ConvArgs a) {
  let_dependents_start();
  wait_for_previous();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= a.total) return;
  for (int token = blockIdx.y; token < a.n; token += gridDim.y) {
    if (c >= a.channels) {
      a.out[static_cast<size_t>(token) * a.total + c] = projected(a, token, c);
      continue;
    }
    const int seq = a.seq_of_token[token];
    const int index = token - a.q_start[seq];
    const int slot = a.state_slot[seq];
    const int T = a.taps_count;
    const bool held = slot >= 0 && slot < a.num_slots;
    const float* state = a.state + static_cast<size_t>(held ? slot : 0) * (T - 1) * a.channels;
    float acc = 0.f;
    for (int j = 0; j < T; ++j) {
      const int lag = T - 1 - j;
      float u;
      if (lag <= index) u = projected(a, token - lag, c);
      else u = held ? state[static_cast<size_t>(T - 1 - (lag - index)) * a.channels + c] : 0.f;
      acc = __fmaf_rn(a.taps[static_cast<size_t>(c) * T + j], u, acc);
    }
    a.out[static_cast<size_t>(token) * a.total + c] = acc;
  }
}

__global__ void __launch_bounds__(256) short_conv_keep_kernel(const ConvArgs a) {
  let_dependents_start();
  wait_for_previous();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int seq = blockIdx.y;
  if (c >= a.channels) return;
  const int slot = a.state_slot[seq];
  if (slot < 0 || slot >= a.num_slots) return;
  const int first = a.q_start[seq], length = a.q_start[seq + 1] - first;
  const int keep = a.taps_count - 1;
  float* state = a.state + static_cast<size_t>(slot) * keep * a.channels;
  float old[MAX_TAPS];
  for (int i = 0; i < keep; ++i) old[i] = i + length < keep ? state[static_cast<size_t>(i + length) * a.channels + c] : 0.f;
  for (int i = 0; i < keep; ++i) {
    const int at = length + i;   // in the old values followed by the portion's
    state[static_cast<size_t>(i) * a.channels + c] = at < keep ? old[i] : projected(a, first + at - keep, c);
  }
}

// ------------------------------------------------------------------------------------------------ gated_scan
constexpr int SCAN_TOKENS = 16;   // tokens staged at a time: their loads are in flight together

struct ScanArgs {
  const float* fused;     // [partials][N][total]: q (H D) | f (H D) | v (H Dv)
  long long stride;
  int partials, total;
  const float* f_bias;    // [H D] or null
  const float* lower;     // [H D] or null: the forget gate's lower bound
  float* state;           // [slots][H][head_stride]: row d, column j of S at d * Dv + j
  const int* q_start;
  const int* state_slot;
  float* out;             // [N][H Dv]
  int heads, dim, vdim, head_stride, cols, row_groups, num_slots;   // row_groups: the lanes of a warp that share a column
  // runs of tokens (0: the whole portion is one walk from the slot's state)
  int run;                // tokens a run holds
  int phase;              // 1: every run from a zero state, leaves its state and its decay; 3: every run from `run_state`
  float* run_state;       // [runs][H][D * Dv]: phase 1 writes a run's own addition, `carry` turns it into the state the run starts from
  float* run_decay;       // [runs][H][D]: the product of a run's forget gates
  int* run_first;         // [S + 1]: index of each sequence's first run; last, the number of runs
  int num_seqs;
  int fast_math;          // 1: the hardware exponential and reciprocal in the gates (a bfloat16 engine)
};

// sigmoid(z) and sigmoid(-z) = 1 - sigmoid(z) from one exponential of -|z| and one reciprocal: neither is formed as a
// difference, so the smaller of the two keeps its digits.  `fast`: the hardware exponential and reciprocal (relative
// error about 2^-21; the bfloat16 engine, whose results keep 8 bits).
__device__ __forceinline__ void sigmoid_both(float z, bool fast, float& with, float& against) {
  const float e = fast ? __expf(-fabsf(z)) : expf(-fabsf(z));             // in (0, 1]
  const float larger = fast ? __fdividef(1.0f, 1.0f + e) : 1.0f / (1.0f + e);   // sigmoid(|z|)
  const float smaller = e * larger;                                       // sigmoid(-|z|)
  with = z >= 0.f ? larger : smaller;
  against = z >= 0.f ? smaller : larger;
}

// One CTA owns `cols` value columns of one head's state for one sequence (or one run of its tokens) and walks the
// tokens in order with the state in registers.  C neighbouring columns are shared by `lanes` neighbouring lanes of a
// warp (a power of two, `row_groups` in the arguments): lane g of them holds rows g R .. g R + R - 1 of those columns,
// so a token costs a thread R C multiply-adds for the state and as many for its share of q . S, what it reads of q, f
// and 1 - f serves C columns, the shares meet by shuffles, and no barrier falls inside the walk.  Tokens are staged
// SCAN_TOKENS at a time: q, f and 1 - f of the head (a lane's rows side by side, each lane's run padded by four floats
// so that the lanes' 16-byte loads fall into different banks) and the CTA's columns of v.
template <int R, int C>
__global__ void __launch_bounds__(C == 1 ? 256 : 128, C == 1 || (R == 32 && C == 2) ? 2 : 4) gated_scan_kernel(const ScanArgs a) {
  extern __shared__ __align__(16) float scan_shared[];
  let_dependents_start();
  wait_for_previous();
  const int D = a.dim, cols = a.cols, lanes = a.row_groups;
  constexpr int PITCH = R + 4;                  // floats between the runs of two neighbouring lanes
  const int padded = lanes * PITCH;             // floats of one staged token's q (or f, or 1 - f)
  float* q = scan_shared;                       // [SCAN_TOKENS][padded]
  float* f = q + SCAN_TOKENS * padded;
  float* k = f + SCAN_TOKENS * padded;          // 1 - f
  float* v = k + SCAN_TOKENS * padded;          // [SCAN_TOKENS][cols]
  float* decay = v + SCAN_TOKENS * cols;        // [D]: phase 1, the product of the run's gates
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane % lanes;
  const int j = (warp * (32 / lanes) + lane / lanes) * C;   // the first of this thread's columns among the CTA's
  const int head = blockIdx.y, col0 = blockIdx.x * cols;
  const int cols_here = min(cols, a.vdim - col0);
  int seq, first, length, run_index = -1;
  if (a.run > 0) {
    // blockIdx.z counts runs over the whole batch: find the sequence
    run_index = blockIdx.z;
    seq = 0;
    while (a.run_first[seq + 1] <= run_index) ++seq;   // run_first[S] is the number of runs; blockIdx.z is below it
    const int within = run_index - a.run_first[seq];
    first = a.q_start[seq] + within * a.run;
    length = min(a.run, a.q_start[seq + 1] - first);
  } else {
    seq = blockIdx.z;
    first = a.q_start[seq];
    length = a.q_start[seq + 1] - first;
  }
  const int slot = a.state_slot[seq];
  const bool held = slot >= 0 && slot < a.num_slots;
  const int HV = a.heads * a.vdim;
  if (!held) {   // a padding row: zeros out, nothing kept
    if (a.phase != 1 && g == 0)
      for (int t = 0; t < length; ++t)
#pragma unroll
        for (int c = 0; c < C; ++c)
          if (j + c < cols_here) a.out[static_cast<size_t>(first + t) * HV + head * a.vdim + col0 + j + c] = 0.f;
    return;
  }
  float* slot_state = a.state + (static_cast<size_t>(slot) * a.heads + head) * a.head_stride;
  float* run_state = a.run > 0 ? a.run_state + (static_cast<size_t>(run_index) * a.heads + head) * D * a.vdim : nullptr;
  const float* from = a.run == 0 ? slot_state : (a.phase == 3 ? run_state : nullptr);
  float S[C][R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int d = g * R + r;
#pragma unroll
    for (int c = 0; c < C; ++c)
      S[c][r] = from != nullptr && j + c < cols_here && d < D ? from[static_cast<size_t>(d) * a.vdim + col0 + j + c] : 0.f;
  }
  // rows past the head's own (the lanes' runs cover lanes * R >= D of them) are zero in q, f and 1 - f, so that the
  // state's rows there stay zero; the four floats between two lanes' runs are never read
  for (int i = threadIdx.x; i < SCAN_TOKENS * (lanes * R - D); i += blockDim.x) {
    const int t = i / (lanes * R - D), d = D + i % (lanes * R - D);
    const int at = t * padded + (d / R) * PITCH + d % R;
    q[at] = 0.f;
    f[at] = 0.f;
    k[at] = 0.f;
  }
  if (a.phase == 1)
    for (int d = threadIdx.x; d < D; d += blockDim.x) decay[d] = 1.f;
  const int q_col = head * D, f_col = a.heads * D + head * D, v_col = 2 * a.heads * D + head * a.vdim + col0;
  for (int t0 = 0; t0 < length; t0 += SCAN_TOKENS) {
    const int here = min(SCAN_TOKENS, length - t0);
    __syncthreads();   // the tokens staged before are used up (and, the first time, the zeros are in place)
#pragma unroll 8
    for (int i = threadIdx.x; i < here * D; i += blockDim.x) {
      const int t = i / D, d = i - t * D;
      const float* row = a.fused + static_cast<size_t>(first + t0 + t) * a.total;
      const float zq = sum_partials(row + q_col + d, a.stride, a.partials);
      float zf = sum_partials(row + f_col + d, a.stride, a.partials);
      if (a.f_bias != nullptr) zf = __fadd_rn(zf, a.f_bias[head * D + d]);
      const float low = a.lower != nullptr ? a.lower[head * D + d] : 0.f;
      const int at = t * padded + (d / R) * PITCH + d % R;
      // 1 - f = (1 - lower) (1 - sigmoid(z)) = (1 - lower) sigmoid(-z): formed so, a gate close to one keeps the
      // digits of what it lets in, which 1 - f computed from f would lose
      float open, shut, q_gate, unused;
      sigmoid_both(zf, a.fast_math != 0, open, shut);
      sigmoid_both(zq, a.fast_math != 0, q_gate, unused);
      q[at] = zq * q_gate;
      f[at] = __fmaf_rn(1.0f - low, open, low);
      k[at] = (1.0f - low) * shut;
    }
#pragma unroll 8
    for (int i = threadIdx.x; i < here * cols; i += blockDim.x) {
      const int t = i / cols, c = i - t * cols;
      v[t * cols + c] = c < cols_here ? sum_partials(a.fused + static_cast<size_t>(first + t0 + t) * a.total + v_col + c, a.stride, a.partials) : 0.f;
    }
    __syncthreads();
    if (a.phase == 1 && blockIdx.x == 0)
      for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float p = decay[d];
        for (int t = 0; t < here; ++t) p *= f[t * padded + (d / R) * PITCH + d % R];
        decay[d] = p;
      }
    for (int t = 0; t < here; ++t) {
      float value[C], partial[C];
#pragma unroll
      for (int c = 0; c < C; ++c) {
        value[c] = v[t * cols + j + c];
        partial[c] = 0.f;
      }
      const float4* f4 = reinterpret_cast<const float4*>(f + t * padded + g * PITCH);
      const float4* k4 = reinterpret_cast<const float4*>(k + t * padded + g * PITCH);
      const float4* q4 = reinterpret_cast<const float4*>(q + t * padded + g * PITCH);
#pragma unroll
      for (int r = 0; r < R; r += 4) {
        const float4 ff = f4[r >> 2], kk = k4[r >> 2], qq = q4[r >> 2];
#pragma unroll
        for (int c = 0; c < C; ++c) {
          S[c][r] = __fmaf_rn(ff.x, S[c][r], kk.x * value[c]);
          S[c][r + 1] = __fmaf_rn(ff.y, S[c][r + 1], kk.y * value[c]);
          S[c][r + 2] = __fmaf_rn(ff.z, S[c][r + 2], kk.z * value[c]);
          S[c][r + 3] = __fmaf_rn(ff.w, S[c][r + 3], kk.w * value[c]);
          partial[c] = __fmaf_rn(S[c][r], qq.x, partial[c]);
          partial[c] = __fmaf_rn(S[c][r + 1], qq.y, partial[c]);
          partial[c] = __fmaf_rn(S[c][r + 2], qq.z, partial[c]);
          partial[c] = __fmaf_rn(S[c][r + 3], qq.w, partial[c]);
        }
      }
      if (a.phase == 1) continue;   // a run's own addition to the state: its outputs come in phase 3
#pragma unroll
      for (int c = 0; c < C; ++c) {
        for (int offset = lanes >> 1; offset > 0; offset >>= 1) partial[c] += __shfl_xor_sync(0xffffffffu, partial[c], offset);
        if (g == 0 && j + c < cols_here) a.out[static_cast<size_t>(first + t0 + t) * HV + head * a.vdim + col0 + j + c] = partial[c];
      }
    }
  }
  if (a.phase == 1) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int d = g * R + r;
#pragma unroll
      for (int c = 0; c < C; ++c)
        if (d < D && j + c < cols_here) run_state[static_cast<size_t>(d) * a.vdim + col0 + j + c] = S[c][r];
    }
    __syncthreads();
    if (blockIdx.x == 0)
      for (int d = threadIdx.x; d < D; d += blockDim.x) a.run_decay[(static_cast<size_t>(run_index) * a.heads + head) * D + d] = decay[d];
    return;
  }
  if (a.run == 0) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int d = g * R + r;
#pragma unroll
      for (int c = 0; c < C; ++c)
        if (d < D && j + c < cols_here) slot_state[static_cast<size_t>(d) * a.vdim + col0 + j + c] = S[c][r];
    }
  }
}

// The index of every sequence's first run, from the batch's lengths: one thread, a few hundred sequences at most.
__global__ void gated_scan_plan_kernel(const ScanArgs a) {
  let_dependents_start();
  wait_for_previous();
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  int runs = 0;
  for (int seq = 0; seq < a.num_seqs; ++seq) {
    a.run_first[seq] = runs;
    runs += (a.q_start[seq + 1] - a.q_start[seq] + a.run - 1) / a.run;
  }
  a.run_first[a.num_seqs] = runs;
}

// The runs' states in order, elementwise: a thread per element of a head's state walks its sequence's runs; where a
// run's own addition was, the state the run starts from is left; the state after the last run goes to the slot.
__global__ void __launch_bounds__(256) gated_scan_carry_kernel(const ScanArgs a) {
  let_dependents_start();
  wait_for_previous();
  const int seq = blockIdx.z, head = blockIdx.y;
  const int element = blockIdx.x * blockDim.x + threadIdx.x;
  const int size = a.dim * a.vdim;
  if (element >= size) return;
  const int slot = a.state_slot[seq];
  if (slot < 0 || slot >= a.num_slots) return;
  const int d = element / a.vdim;
  float* slot_state = a.state + (static_cast<size_t>(slot) * a.heads + head) * a.head_stride + element;
  float s = *slot_state;
  const int last = a.run_first[seq + 1];
  // eight runs' additions and decays are asked for together: the walk is one memory latency per eight runs
  for (int run0 = a.run_first[seq]; run0 < last; run0 += 8) {
    float added[8], p[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const size_t at = static_cast<size_t>(min(run0 + i, last - 1)) * a.heads + head;
      added[i] = a.run_state[at * size + element];
      p[i] = a.run_decay[at * a.dim + d];
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (run0 + i < last) {
        a.run_state[(static_cast<size_t>(run0 + i) * a.heads + head) * size + element] = s;
        s = __fmaf_rn(p[i], s, added[i]);
      }
    }
  }
  *slot_state = s;
}

// ------------------------------------------------------------------------------------------------ head_rms
template <typename TO>
__global__ void __launch_bounds__(128) head_rms_kernel(const float* __restrict__ x, const float* __restrict__ weight,
                                                       TO* __restrict__ out, int n, int heads, int size, float eps) {
  let_dependents_start();
  wait_for_previous();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long unit = static_cast<long long>(blockIdx.x) * 4 + warp;
  if (unit >= static_cast<long long>(n) * heads) return;
  const float* row = x + unit * size;
  float squares = 0.f;
  for (int d = lane; d < size; d += 32) squares = __fmaf_rn(row[d], row[d], squares);
  const float r = rsqrtf(warp_sum(squares) / static_cast<float>(size) + eps);
  for (int d = lane; d < size; d += 32) out[unit * size + d] = from_float<TO>(row[d] * r * (weight != nullptr ? weight[d] : 1.f));
}

}  // namespace streams

// =========================================================================================== launchers
using namespace streams;

// terms: `num_terms` (at most 4) pending sums, term t = data[t] ([partials[t]][N][W] float32, `strides[t]` elements
// between partials) times scales[t]; they join the streams only when `mix` is given.  out_dtype: the type of `out`.
SHRIKE_API int shrike_stream_norm(float* x, const float* const* data, const int* partials, const long long* strides,
                                  const float* scales, int num_terms, const float* mix, const float* out_w,
                                  const float* layer_scale, const float* in_w, const float* norm_w, float eps, void* out,
                                  int out_dtype, float* sum_out, const int* rows, int n, int width, int count,
                                  cudaStream_t stream) {
  if (n <= 0) return SHRIKE_OK;
  if (width < 1 || count < 1 || count > MAX_STREAMS || num_terms < 0 || num_terms > MAX_TERMS) return SHRIKE_BAD_ARGUMENT;
  if (mix != nullptr && out_w == nullptr) return SHRIKE_BAD_ARGUMENT;
  StreamNormArgs a = {};
  a.x = x;
  a.num_terms = mix != nullptr ? num_terms : 0;
  bool vec = width % 4 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0 &&
             reinterpret_cast<uintptr_t>(norm_w) % 16 == 0;
  for (int t = 0; t < a.num_terms; ++t) {
    if (data[t] == nullptr || partials[t] < 1) return SHRIKE_BAD_ARGUMENT;
    a.terms[t] = {data[t], strides[t], partials[t], scales[t]};
    vec = vec && reinterpret_cast<uintptr_t>(data[t]) % 16 == 0 && strides[t] % 4 == 0;
  }
  a.mix = mix; a.out_w = out_w; a.layer_scale = layer_scale; a.in_w = in_w; a.norm_w = norm_w; a.eps = eps;
  a.out = out; a.sum_out = sum_out; a.rows = rows; a.n = n; a.width = width; a.count = count;
  // few rows (a decode step, the final norm's wanted rows): a row's columns go to the CTAs of a cluster, as many as
  // leave every CTA a few hundred columns
  a.split = 1;
  if (n <= 64 && norm_w != nullptr && out != nullptr)
    while (a.split < 8 && width / (vec ? 4 : 1) / (a.split * 2) >= 64) a.split *= 2;
  const size_t smem = (static_cast<size_t>(width) + 33) * sizeof(float);
  if (smem > static_cast<size_t>(shrike_device().max_smem)) return SHRIKE_BAD_ARGUMENT;
  const bool bf16 = out != nullptr && out_dtype == SHRIKE_BF16;
  if (out != nullptr && out_dtype != SHRIKE_BF16 && out_dtype != SHRIKE_F32) return SHRIKE_BAD_ARGUMENT;
  const unsigned grid = static_cast<unsigned>(n) * static_cast<unsigned>(a.split);
#define SHRIKE_STREAM_LAUNCH(T, V, M)                                                                                   \
  do {                                                                                                                  \
    if (smem > 48 * 1024)                                                                                               \
      cudaFuncSetAttribute(stream_norm_kernel<T, V, M>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)); \
    if (a.split > 1) launch_dependent_clusters(stream_norm_kernel<T, V, M>, grid, 256, smem, stream, a.split, a);       \
    else launch_dependent(stream_norm_kernel<T, V, M>, grid, 256, smem, stream, a);                                     \
  } while (0)
#define SHRIKE_STREAM_CASE(T, V)                                                                                        \
  do {                                                                                                                  \
    if (count <= 1) SHRIKE_STREAM_LAUNCH(T, V, 1);                                                                      \
    else if (count <= 2) SHRIKE_STREAM_LAUNCH(T, V, 2);                                                                 \
    else if (count <= 4) SHRIKE_STREAM_LAUNCH(T, V, 4);                                                                 \
    else SHRIKE_STREAM_LAUNCH(T, V, 8);                                                                                 \
  } while (0)
  if (bf16 && vec) SHRIKE_STREAM_CASE(__nv_bfloat16, 4);
  else if (bf16) SHRIKE_STREAM_CASE(__nv_bfloat16, 1);
  else if (vec) SHRIKE_STREAM_CASE(float, 4);
  else SHRIKE_STREAM_CASE(float, 1);
#undef SHRIKE_STREAM_LAUNCH
#undef SHRIKE_STREAM_CASE
  return shrike_launch_status();
}

// Two launches: the convolution (every token and channel by itself), then the state (a thread a sequence and channel).
SHRIKE_API int shrike_short_conv(const float* fused, int partials, long long stride, int total, const float* bias,
                                 const float* taps, float* state, const int* q_start, const int* state_slot,
                                 const int* seq_of_token, float* out, int n, int channels, int taps_count, int num_seqs,
                                 int num_slots, cudaStream_t stream) {
  if (n <= 0) return SHRIKE_OK;
  if (channels < 1 || channels > total || taps_count < 1 || taps_count > MAX_TAPS || partials < 1 || num_seqs < 1 || num_seqs > 65535)
    return SHRIKE_BAD_ARGUMENT;
  ConvArgs a = {fused, stride, partials, total, bias, taps, state, q_start, state_slot, seq_of_token, out,
                n, channels, taps_count, num_seqs, num_slots};
  const dim3 grid(static_cast<unsigned>((total + 255) / 256), static_cast<unsigned>(min(n, 65535)));
  launch_dependent(short_conv_kernel, grid, 256, 0, stream, a);
  if (taps_count > 1) {
    const dim3 keep(static_cast<unsigned>((channels + 255) / 256), static_cast<unsigned>(num_seqs));
    launch_dependent(short_conv_keep_kernel, keep, 256, 0, stream, a);
  }
  return shrike_launch_status();
}

// How the scan is laid out for heads of dim x vdim: R rows of C neighbouring columns a thread, the lanes that share
// those columns (a power of two covering dim), the columns a CTA of up to four warps takes.  `wide` (16 x 4; 8 x 4 for
// heads of up to 32 rows, 32 x 2 above 512): what a thread reads of q, f and 1 - f serves four columns, which is what
// bounds a walk when there is enough of it to fill the GPU; otherwise one column a thread (32 x 1, 8 x 1), twice to four
// times the threads for the same state.
struct ScanShape { int rows, each, lanes, cols, threads; size_t smem; };
static inline bool scan_shape(int dim, int vdim, bool wide, ScanShape* shape) {
  int rows, each;
  if (dim <= 32) { rows = 8; each = wide ? 4 : 1; }
  else if (dim <= 512 && wide) { rows = 16; each = 4; }
  else { rows = 32; each = wide ? 2 : 1; }
  int lanes = 1;
  while (lanes * rows < dim) lanes *= 2;
  if (lanes > 32) return false;
  const int per_warp = 32 / lanes * each;
  const int warps = max(1, min(each == 1 ? 8 : 4, (vdim + per_warp - 1) / per_warp));   // either way up to 64 columns a CTA at 128 rows
  shape->rows = rows; shape->each = each; shape->lanes = lanes; shape->cols = per_warp * warps; shape->threads = warps * 32;
  shape->smem = (static_cast<size_t>(3) * SCAN_TOKENS * lanes * (rows + 4) + static_cast<size_t>(SCAN_TOKENS) * shape->cols + dim) * sizeof(float);
  return shape->smem <= static_cast<size_t>(shrike_device().max_smem);
}

SHRIKE_API long long shrike_gated_scan_runs(int n, int num_seqs, int run) { return (static_cast<long long>(n) + run - 1) / run + num_seqs; }

// `run` > 0: portions are cut into runs of that many tokens, which walk side by side (three launches); `run_state`
// (runs x heads x dim x vdim floats), `run_decay` (runs x heads x dim) and `run_first` (int32 [S + 1] of scratch: a
// first launch leaves the index of every sequence's first run there) are then needed, and `num_runs` is the number
// of runs the batch's lengths make, the sum of ceil(length / run).
SHRIKE_API int shrike_gated_scan(const float* fused, int partials, long long stride, int total, const float* f_bias,
                                 const float* lower, float* state, const int* q_start, const int* state_slot, float* out,
                                 int num_seqs, int heads, int dim, int vdim, int head_stride, int num_slots, int run,
                                 float* run_state, float* run_decay, int* run_first, int num_runs, int fast_math,
                                 cudaStream_t stream) {
  if (num_seqs <= 0) return SHRIKE_OK;
  if (heads < 1 || heads > 65535 || num_seqs > 65535 || dim < 1 || vdim < 1 || partials < 1 || head_stride < dim * vdim ||
      total < heads * (2 * dim + vdim))
    return SHRIKE_BAD_ARGUMENT;
  // the wide form where the walks fill the GPU with it (about three warps a sub-partition), else one column a thread
  const bool runs = run > 0 && run_state != nullptr && run_decay != nullptr && run_first != nullptr && num_runs >= 1;
  ScanShape shape;
  if (!scan_shape(dim, vdim, true, &shape)) return SHRIKE_BAD_ARGUMENT;   // heads of more than 1,024 rows
  const long long wide_threads = static_cast<long long>(heads) * (runs ? num_runs : num_seqs) * ((vdim + shape.each - 1) / shape.each) * shape.lanes;
  if (wide_threads < static_cast<long long>(shrike_device().sm_count) * 384 && !scan_shape(dim, vdim, false, &shape)) return SHRIKE_BAD_ARGUMENT;
  ScanArgs a = {fused, stride, partials, total, f_bias, lower, state, q_start, state_slot, out, heads, dim, vdim,
                head_stride, shape.cols, shape.lanes, num_slots, 0, 0, nullptr, nullptr, nullptr, num_seqs, fast_math};
  void (*kernel)(ScanArgs) = nullptr;
  if (shape.rows == 8) kernel = shape.each == 4 ? gated_scan_kernel<8, 4> : gated_scan_kernel<8, 1>;
  else if (shape.rows == 16) kernel = gated_scan_kernel<16, 4>;
  else kernel = shape.each == 2 ? gated_scan_kernel<32, 2> : gated_scan_kernel<32, 1>;
  if (shape.smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(shape.smem));
  const unsigned slices = static_cast<unsigned>((vdim + shape.cols - 1) / shape.cols);
  const unsigned threads = static_cast<unsigned>(shape.threads);
  if (!runs) {
    launch_dependent(kernel, dim3(slices, heads, num_seqs), threads, shape.smem, stream, a);
    return shrike_launch_status();
  }
  if (num_runs > 65535) return SHRIKE_BAD_ARGUMENT;
  a.run = run; a.run_state = run_state; a.run_decay = run_decay; a.run_first = run_first;
  launch_dependent(gated_scan_plan_kernel, 1, 32, 0, stream, a);
  a.phase = 1;
  launch_dependent(kernel, dim3(slices, heads, num_runs), threads, shape.smem, stream, a);
  launch_dependent(gated_scan_carry_kernel, dim3((dim * vdim + 255) / 256, heads, num_seqs), 256, 0, stream, a);
  a.phase = 3;
  launch_dependent(kernel, dim3(slices, heads, num_runs), threads, shape.smem, stream, a);
  return shrike_launch_status();
}

SHRIKE_API int shrike_head_rms(const float* x, const float* weight, void* out, int dtype, int n, int heads, int size,
                               float eps, cudaStream_t stream) {
  if (n <= 0) return SHRIKE_OK;
  if (heads < 1 || size < 1) return SHRIKE_BAD_ARGUMENT;
  const long long units = static_cast<long long>(n) * heads;
  const long long blocks = (units + 3) / 4;
  if (blocks > 0x7fffffffLL) return SHRIKE_BAD_ARGUMENT;
  if (dtype == SHRIKE_F32)
    launch_dependent(head_rms_kernel<float>, static_cast<unsigned>(blocks), 128, 0, stream, x, weight, static_cast<float*>(out), n, heads, size, eps);
  else if (dtype == SHRIKE_BF16)
    launch_dependent(head_rms_kernel<__nv_bfloat16>, static_cast<unsigned>(blocks), 128, 0, stream, x, weight,
                     static_cast<__nv_bfloat16*>(out), n, heads, size, eps);
  else return SHRIKE_BAD_ARGUMENT;
  return shrike_launch_status();
}
