// Kernels of the decayed linear attention and of the latent attention with a rotated key part, and two
// small ones that other parts share:
//
//   decay_scan         S_t = d S_(t-1) + k_t v_t^T, o_t = S_t^T q_t per head over the batch's new tokens, with
//                      q, k, v = silu of columns of a fused projection; the state is read from and left in
//                      the request's slot.  Single tokens and short portions walk token by token with the
//                      state in registers; long portions run in three launches over runs of 64 tokens
//                      (`chunk_local`, `chunk_carry`, `chunk_finish`), the same sum in another order.
//   norm_gate          rows divided by their root mean square and scaled by a weight (optional), times the
//                      sigmoid of columns of a fused projection (optional), cast to the engine's type
//   latent_rope_store  queries, latent and shared key part of a fused projection: the latent normed, the
//                      rotated parts turned by position, queries cast, the token's page row written
//   concat_cast        pending sums added to the float32 residual, then [residual | other] side by side in
//                      the engine's type: the input of a product over both
//
// Everything that enters the recurrence (activations, decays and their powers, the state) and every norm is
// float32.  A fused projection may come as a stack of K-split partial sums, which are added on the fly.
#include "common.cuh"

namespace decay {

constexpr int THREADS = 256;
constexpr int MAX_SLICE = 64;   // columns of a head's state one CTA holds
constexpr int CHUNK = 64;       // tokens of a run in the chunked form

__device__ __forceinline__ float silu(float z) { return z / (1.0f + expf(-z)); }

// d^n for an integer n >= 0 by squaring: the same bits wherever it is formed
__device__ __forceinline__ float int_power(float d, int n) {
  float result = 1.0f, base = d;
  while (n > 0) {
    if (n & 1) result *= base;
    base *= base;
    n >>= 1;
  }
  return result;
}

struct ScanArgs {
  const float* fused;       // [partials][n][row_width]
  int partials;
  long long partial_stride;
  int row_width;
  const float* decays;      // [heads]
  float* state;             // [slots][heads][state_stride]
  const int* q_start;       // [seqs + 1]
  const int* state_slot;    // [seqs]
  float* out;               // [n][heads * vdim]
  int heads, dim, vdim, num_slots, state_stride;
  int slice;                // columns per CTA
  int groups;               // row groups per CTA: thread t owns column t % slice, rows t / slice + i * groups
};

// Walk: grid (vdim slices, heads, seqs).  Each thread keeps ROWS elements of the state in registers.
template <int ROWS>
__global__ void __launch_bounds__(THREADS) walk_kernel(ScanArgs a, int skip_longer_than) {
  extern __shared__ __align__(16) float shared[];
  float* q_s = shared;                    // [dim]
  float* k_s = q_s + a.dim;               // [dim]
  float* v_s = k_s + a.dim;               // [slice]
  float* part = v_s + a.slice;            // [groups][slice]
  let_dependents_start();
  wait_for_previous();
  const int seq = blockIdx.z, head = blockIdx.y, first_col = blockIdx.x * a.slice;
  const int slot = a.state_slot[seq];
  if (slot < 0 || slot >= a.num_slots) return;
  const int begin = a.q_start[seq], end = a.q_start[seq + 1];
  if (skip_longer_than > 0 && end - begin > skip_longer_than) return;   // the chunked form serves it
  const int cols = min(a.slice, a.vdim - first_col);
  const int t = threadIdx.x;
  const int col = t % a.slice, group = t / a.slice;
  const bool active = group < a.groups && col < cols;
  const float d = a.decays[head];
  float* mine = a.state + (static_cast<size_t>(slot) * a.heads + head) * a.state_stride;
  float held[ROWS];
#pragma unroll
  for (int i = 0; i < ROWS; ++i) {
    const int row = group + i * a.groups;
    held[i] = active && row < a.dim ? mine[static_cast<size_t>(row) * a.vdim + first_col + col] : 0.f;
  }
  const int q_at = head * a.dim, k_at = a.heads * a.dim + head * a.dim, v_at = 2 * a.heads * a.dim + head * a.vdim + first_col;
  for (int token = begin; token < end; ++token) {
    const float* row = a.fused + static_cast<size_t>(token) * a.row_width;
    for (int i = t; i < 2 * a.dim + cols; i += THREADS) {
      const int at = i < a.dim ? q_at + i : (i < 2 * a.dim ? k_at + i - a.dim : v_at + i - 2 * a.dim);
      q_s[i] = silu(sum_partials(row + at, a.partial_stride, a.partials));   // q_s, k_s and v_s lie one after the other
    }
    __syncthreads();
    float sum = 0.f;
    if (active) {
      const float v = v_s[col];
#pragma unroll
      for (int i = 0; i < ROWS; ++i) {
        const int r = group + i * a.groups;
        if (r < a.dim) {
          held[i] = fmaf(d, held[i], k_s[r] * v);
          sum = fmaf(held[i], q_s[r], sum);
        }
      }
      part[group * a.slice + col] = sum;
    }
    __syncthreads();
    if (t < cols) {
      float total = 0.f;
      for (int g = 0; g < a.groups; ++g) total += part[g * a.slice + t];
      a.out[static_cast<size_t>(token) * a.heads * a.vdim + head * a.vdim + first_col + t] = total;
    }
  }
#pragma unroll
  for (int i = 0; i < ROWS; ++i) {
    const int row = group + i * a.groups;
    if (active && row < a.dim) mine[static_cast<size_t>(row) * a.vdim + first_col + col] = held[i];
  }
}

// The same walk for heads of so many rows that a thread's share of the state does not fit its registers: the state
// stays in memory and every token reads and rewrites it (slow, and right; no model of the usual sizes comes here).
__global__ void __launch_bounds__(THREADS) walk_in_memory_kernel(ScanArgs a, int skip_longer_than) {
  extern __shared__ __align__(16) float shared[];
  float* q_s = shared;                    // [dim]
  float* k_s = q_s + a.dim;               // [dim]
  float* v_s = k_s + a.dim;               // [slice]
  float* part = v_s + a.slice;            // [groups][slice]
  let_dependents_start();
  wait_for_previous();
  const int seq = blockIdx.z, head = blockIdx.y, first_col = blockIdx.x * a.slice;
  const int slot = a.state_slot[seq];
  if (slot < 0 || slot >= a.num_slots) return;
  const int begin = a.q_start[seq], end = a.q_start[seq + 1];
  if (skip_longer_than > 0 && end - begin > skip_longer_than) return;   // the chunked form serves it
  const int cols = min(a.slice, a.vdim - first_col);
  const int t = threadIdx.x;
  const int col = t % a.slice, group = t / a.slice;
  const bool active = group < a.groups && col < cols;
  const float d = a.decays[head];
  float* mine = a.state + (static_cast<size_t>(slot) * a.heads + head) * a.state_stride + first_col + col;
  const int q_at = head * a.dim, k_at = a.heads * a.dim + head * a.dim, v_at = 2 * a.heads * a.dim + head * a.vdim + first_col;
  for (int token = begin; token < end; ++token) {
    const float* row = a.fused + static_cast<size_t>(token) * a.row_width;
    __syncthreads();   // the token before is done with q_s and part
    for (int i = t; i < 2 * a.dim + cols; i += THREADS) {
      const int at = i < a.dim ? q_at + i : (i < 2 * a.dim ? k_at + i - a.dim : v_at + i - 2 * a.dim);
      q_s[i] = silu(sum_partials(row + at, a.partial_stride, a.partials));
    }
    __syncthreads();
    if (active) {
      const float v = v_s[col];
      float sum = 0.f;
      for (int r = group; r < a.dim; r += a.groups) {   // the same rows, in the same order, as the walk in registers
        float* at = mine + static_cast<size_t>(r) * a.vdim;
        const float held = fmaf(d, *at, k_s[r] * v);
        *at = held;
        sum = fmaf(held, q_s[r], sum);
      }
      part[group * a.slice + col] = sum;
    }
    __syncthreads();
    if (t < cols) {
      float total = 0.f;
      for (int g = 0; g < a.groups; ++g) total += part[g * a.slice + t];
      a.out[static_cast<size_t>(token) * a.heads * a.vdim + head * a.vdim + first_col + t] = total;
    }
  }
}

// ---- the chunked form ---------------------------------------------------------------------------------------
// A sequence's new tokens are cut into runs of CHUNK from its first new token; only sequences that bring more than
// `skip` tokens have runs, numbered sequence by sequence.  Every CTA finds its run from `q_start` alone (a walk over
// the batch's sequences), so the launches depend on the batch's shape only.  For run c with tokens a .. b of a head
// with decay d:
//   local   L_c = sum_j d^(b - j) k_j v_j^T  and  o_t = sum_(a <= j <= t) d^(t - j) (q_t . k_j) v_j
//   carry   S_after(c) = d^(b - a + 1) S_before(c) + L_c, run after run of a sequence; S_before kept per run
//   finish  o_t += d^(t - a + 1) S_before(c)^T q_t
struct ChunkArgs {
  ScanArgs s;
  float* chunk_state;       // [runs][heads][dim * vdim]: L_c, then S_before(c)
  int num_seqs;
  int skip;                 // sequences of at most this many new tokens have no runs (they walk)
  int span;                 // value columns one CTA of `local` and `finish` serves, a multiple of MAX_SLICE
};

// Run number `run` of the batch: its sequence, first token and token count.  False: there is no such run.
__device__ __forceinline__ bool locate_run(const ChunkArgs& c, int run, int& seq, int& first, int& count) {
  int before = 0;
  for (int s = 0; s < c.num_seqs; ++s) {
    const int begin = c.s.q_start[s], length = c.s.q_start[s + 1] - begin;
    const int runs = length > c.skip ? (length + CHUNK - 1) / CHUNK : 0;
    if (run < before + runs) {
      const int index = run - before;
      seq = s;
      first = begin + index * CHUNK;
      count = min(CHUNK, length - index * CHUNK);
      return true;
    }
    before += runs;
  }
  return false;
}

// The three products of a run (scores, scores times values, keys times values) and the product of `finish` run as
// register tiles over shared memory: 256 threads as 16 x 16, thread (ty, tx) owning rows ty + 16 r and either rows
// tx + 16 c of the other operand (scores) or columns 4 tx .. 4 tx + 3 (the others), four reduction steps a 16-byte load.
// Rows of q and k are padded to `chunk_pitch` floats, a multiple of four whose quarter is odd: the sixteen rows a
// half-warp reads at once fall into different banks.
__host__ __device__ __forceinline__ int chunk_pitch(int dim) { return ((dim + 7) & ~7) + 4; }
constexpr int SCORE_PITCH = CHUNK + 4;

__device__ __forceinline__ void fma4(float (&acc)[4], float w, const float4& v) {
  acc[0] = fmaf(w, v.x, acc[0]); acc[1] = fmaf(w, v.y, acc[1]); acc[2] = fmaf(w, v.z, acc[2]); acc[3] = fmaf(w, v.w, acc[3]);
}

// silu of columns [at, at + width) of the fused projection for tokens first .. first + count - 1 into dst[j * pitch + e];
// rows from `count` on and columns from `width` to `fill_to` are zero
__device__ __forceinline__ void stage_rows(float* dst, int pitch, int fill_to, const ScanArgs& a, int first, int count, int at,
                                           int width) {
  const bool wide = a.partials == 1 && (width & 3) == 0 && (fill_to & 3) == 0 && (at & 3) == 0 && (a.row_width & 3) == 0 &&
                    (reinterpret_cast<uintptr_t>(a.fused) & 15) == 0;
  if (wide) {
    const int quads = fill_to >> 2;
    for (int i = threadIdx.x; i < CHUNK * quads; i += THREADS) {
      const int j = i / quads, e = (i - j * quads) << 2;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (j < count && e < width) {
        v = *reinterpret_cast<const float4*>(a.fused + static_cast<size_t>(first + j) * a.row_width + at + e);
        v.x = silu(v.x); v.y = silu(v.y); v.z = silu(v.z); v.w = silu(v.w);
      }
      *reinterpret_cast<float4*>(dst + j * pitch + e) = v;
    }
    return;
  }
  for (int i = threadIdx.x; i < CHUNK * fill_to; i += THREADS) {
    const int j = i / fill_to, e = i - j * fill_to;
    float v = 0.f;
    if (j < count && e < width)
      v = silu(sum_partials(a.fused + static_cast<size_t>(first + j) * a.row_width + at + e, a.partial_stride, a.partials));
    dst[j * pitch + e] = v;
  }
}

// grid (column groups of `span`, heads, runs): intra-run outputs and L_c, 64 columns at a time.
__global__ void __launch_bounds__(THREADS) chunk_local_kernel(ChunkArgs c) {
  extern __shared__ __align__(16) float shared[];
  const ScanArgs& a = c.s;
  const int pitch = chunk_pitch(a.dim), dim8 = (a.dim + 7) & ~7, dim4 = (a.dim + 3) & ~3;
  float* q_s = shared;                              // [CHUNK][pitch]
  float* k_s = q_s + CHUNK * pitch;                 // [CHUNK][pitch]
  float* v_s = k_s + CHUNK * pitch;                 // [CHUNK][MAX_SLICE]
  float* w_s = v_s + CHUNK * MAX_SLICE;             // [CHUNK][SCORE_PITCH] decayed scores, zero above the diagonal
  float* pow_s = w_s + CHUNK * SCORE_PITCH;         // [CHUNK + 1] d^n
  let_dependents_start();
  wait_for_previous();
  const int run = blockIdx.z, head = blockIdx.y;
  int seq, first, count;
  if (!locate_run(c, run, seq, first, count)) return;
  const int slot = a.state_slot[seq];
  if (slot < 0 || slot >= a.num_slots) return;
  const int t = threadIdx.x, tx = t & 15, ty = t >> 4;
  const float d = a.decays[head];
  const int q_at = head * a.dim, k_at = a.heads * a.dim + head * a.dim;
  stage_rows(q_s, pitch, dim8, a, first, count, q_at, a.dim);
  stage_rows(k_s, pitch, dim8, a, first, count, k_at, a.dim);
  for (int n = t; n <= CHUNK; n += THREADS) pow_s[n] = int_power(d, n);
  __syncthreads();
  {   // decayed scores w[i][j] = d^(i - j) q_i . k_j for j <= i: rows ty + 16 r, keys tx + 16 c, only c <= r can be seen
    float acc[4][4] = {};
    for (int e = 0; e < dim4; e += 4) {
      float4 qv[4], kv[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) qv[r] = *reinterpret_cast<const float4*>(q_s + (ty + 16 * r) * pitch + e);
#pragma unroll
      for (int r = 0; r < 4; ++r) kv[r] = *reinterpret_cast<const float4*>(k_s + (tx + 16 * r) * pitch + e);
#pragma unroll
      for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int cc = 0; cc <= r; ++cc) {
          acc[r][cc] = fmaf(qv[r].x, kv[cc].x, acc[r][cc]);
          acc[r][cc] = fmaf(qv[r].y, kv[cc].y, acc[r][cc]);
          acc[r][cc] = fmaf(qv[r].z, kv[cc].z, acc[r][cc]);
          acc[r][cc] = fmaf(qv[r].w, kv[cc].w, acc[r][cc]);
        }
    }
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) {
        const int qi = ty + 16 * r, kj = tx + 16 * cc;
        w_s[qi * SCORE_PITCH + kj] = (cc <= r && kj <= qi && qi < count) ? acc[r][cc] * pow_s[qi - kj] : 0.f;
      }
  }
  const int v_first = 2 * a.heads * a.dim + head * a.vdim;
  const size_t out_pitch = static_cast<size_t>(a.heads) * a.vdim;
  const bool wide_out = (a.vdim & 3) == 0;
  float* local = c.chunk_state + (static_cast<size_t>(run) * a.heads + head) * a.dim * a.vdim;
  const int last_col = min(a.vdim, (static_cast<int>(blockIdx.x) + 1) * c.span);
  for (int first_col = blockIdx.x * c.span; first_col < last_col; first_col += MAX_SLICE) {
    const int cols = min(MAX_SLICE, a.vdim - first_col);
    __syncthreads();   // the scores are whole; the pass before is done with v_s
    stage_rows(v_s, MAX_SLICE, MAX_SLICE, a, first, count, v_first + first_col, cols);
    __syncthreads();
    {   // o_i = sum_(j <= i) w[i][j] v_j: rows ty + 16 r, columns 4 tx .., keys sixteen at a time (block jb reaches rows r >= jb)
      float o[4][4] = {};
#pragma unroll
      for (int jb = 0; jb < 4; ++jb) {
        if (16 * jb >= count) break;
#pragma unroll
        for (int j = 16 * jb; j < 16 * jb + 16; j += 4) {
          float4 vv[4];
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) vv[kk] = *reinterpret_cast<const float4*>(v_s + (j + kk) * MAX_SLICE + 4 * tx);
#pragma unroll
          for (int r = jb; r < 4; ++r) {
            const float4 w = *reinterpret_cast<const float4*>(w_s + (ty + 16 * r) * SCORE_PITCH + j);
            fma4(o[r], w.x, vv[0]); fma4(o[r], w.y, vv[1]); fma4(o[r], w.z, vv[2]); fma4(o[r], w.w, vv[3]);
          }
        }
      }
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int qi = ty + 16 * r;
        if (qi >= count) continue;
        float* dst = a.out + static_cast<size_t>(first + qi) * out_pitch + head * a.vdim + first_col + 4 * tx;
        if (wide_out) {
          if (4 * tx < cols) *reinterpret_cast<float4*>(dst) = make_float4(o[r][0], o[r][1], o[r][2], o[r][3]);
        } else {
#pragma unroll
          for (int e = 0; e < 4; ++e)
            if (4 * tx + e < cols) dst[e] = o[r][e];
        }
      }
    }
    // L_c[r][e] = sum_j d^(count - 1 - j) k_j[r] v_j[e]: rows 8 ty .. 8 ty + 7 of 128 at a time, columns 4 tx ..
    for (int base = 0; base < a.dim; base += 128) {
      const int r0 = base + 8 * ty;
      if (r0 >= a.dim) continue;
      float l[8][4] = {};
      for (int j = 0; j < count; ++j) {
        float4 v = *reinterpret_cast<const float4*>(v_s + j * MAX_SLICE + 4 * tx);
        const float p = pow_s[count - 1 - j];
        v.x *= p; v.y *= p; v.z *= p; v.w *= p;
        const float4 k0 = *reinterpret_cast<const float4*>(k_s + j * pitch + r0);
        const float4 k1 = *reinterpret_cast<const float4*>(k_s + j * pitch + r0 + 4);
        fma4(l[0], k0.x, v); fma4(l[1], k0.y, v); fma4(l[2], k0.z, v); fma4(l[3], k0.w, v);
        fma4(l[4], k1.x, v); fma4(l[5], k1.y, v); fma4(l[6], k1.z, v); fma4(l[7], k1.w, v);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (r0 + i >= a.dim) continue;
        float* dst = local + static_cast<size_t>(r0 + i) * a.vdim + first_col + 4 * tx;
        if (wide_out) {
          if (4 * tx < cols) *reinterpret_cast<float4*>(dst) = make_float4(l[i][0], l[i][1], l[i][2], l[i][3]);
        } else {
#pragma unroll
          for (int e = 0; e < 4; ++e)
            if (4 * tx + e < cols) dst[e] = l[i][e];
        }
      }
    }
  }
}

// grid (blocks over dim * vdim / VEC, heads, seqs): walks a sequence's runs in order, VEC elements a thread; the
// additions of eight runs are asked for together, so that a sequence costs a memory latency every eight runs.
constexpr int CARRY_AHEAD = 8;

template <int VEC>
__global__ void __launch_bounds__(THREADS) chunk_carry_kernel(ChunkArgs c) {
  const ScanArgs& a = c.s;
  let_dependents_start();
  wait_for_previous();
  const int seq = blockIdx.z, head = blockIdx.y;
  const int slot = a.state_slot[seq];
  if (slot < 0 || slot >= a.num_slots) return;
  const int length = a.q_start[seq + 1] - a.q_start[seq];
  if (length <= c.skip) return;   // the walk serves it
  const int element = (blockIdx.x * THREADS + threadIdx.x) * VEC;
  if (element >= a.dim * a.vdim) return;
  int run = 0;   // the sequence's first run: those of the sequences before it come first
  for (int s = 0; s < seq; ++s) {
    const int other = a.q_start[s + 1] - a.q_start[s];
    if (other > c.skip) run += (other + CHUNK - 1) / CHUNK;
  }
  const float d = a.decays[head];
  const float whole = int_power(d, CHUNK);
  float* mine = a.state + (static_cast<size_t>(slot) * a.heads + head) * a.state_stride + element;
  const size_t per_run = static_cast<size_t>(a.heads) * a.dim * a.vdim;
  float* local = c.chunk_state + (static_cast<size_t>(run) * a.heads + head) * a.dim * a.vdim + element;
  const int runs = (length + CHUNK - 1) / CHUNK;
  float held[VEC];
  if constexpr (VEC == 4) load4<float>(mine, held);
  else held[0] = *mine;
  for (int r = 0; r < runs; r += CARRY_AHEAD) {
    float add[CARRY_AHEAD][VEC];
#pragma unroll
    for (int i = 0; i < CARRY_AHEAD; ++i)
      if (r + i < runs) {
        if constexpr (VEC == 4) load4<float>(local + (r + i) * per_run, add[i]);
        else add[i][0] = local[(r + i) * per_run];
      }
#pragma unroll
    for (int i = 0; i < CARRY_AHEAD; ++i)
      if (r + i < runs) {
        float* at = local + (r + i) * per_run;       // S before this run: what `finish` reads
        if constexpr (VEC == 4) *reinterpret_cast<float4*>(at) = make_float4(held[0], held[1], held[2], held[3]);
        else *at = held[0];
        const int tokens = min(CHUNK, length - (r + i) * CHUNK);
        const float keep = tokens == CHUNK ? whole : int_power(d, tokens);
#pragma unroll
        for (int e = 0; e < VEC; ++e) held[e] = fmaf(keep, held[e], add[i][e]);
      }
  }
  if constexpr (VEC == 4) *reinterpret_cast<float4*>(mine) = make_float4(held[0], held[1], held[2], held[3]);
  else *mine = held[0];
}

// grid (column groups of `span`, heads, runs): o_t += d^(t - a + 1) S_before^T q_t, 64 columns at a time.
__global__ void __launch_bounds__(THREADS) chunk_finish_kernel(ChunkArgs c) {
  extern __shared__ __align__(16) float shared[];
  const ScanArgs& a = c.s;
  const int pitch = chunk_pitch(a.dim), dim4 = (a.dim + 3) & ~3;
  float* q_s = shared;                        // [CHUNK][pitch]
  float* s_s = q_s + CHUNK * pitch;           // [dim4][MAX_SLICE]
  float* pow_s = s_s + dim4 * MAX_SLICE;      // [CHUNK + 1]
  let_dependents_start();
  wait_for_previous();
  const int run = blockIdx.z, head = blockIdx.y;
  int seq, first, count;
  if (!locate_run(c, run, seq, first, count)) return;
  const int slot = a.state_slot[seq];
  if (slot < 0 || slot >= a.num_slots) return;
  const int t = threadIdx.x, tx = t & 15, ty = t >> 4;
  const float d = a.decays[head];
  stage_rows(q_s, pitch, (a.dim + 7) & ~7, a, first, count, head * a.dim, a.dim);
  for (int n = t; n <= CHUNK; n += THREADS) pow_s[n] = int_power(d, n);
  const float* before = c.chunk_state + (static_cast<size_t>(run) * a.heads + head) * a.dim * a.vdim;
  const size_t out_pitch = static_cast<size_t>(a.heads) * a.vdim;
  const bool wide = (a.vdim & 3) == 0;
  const int last_col = min(a.vdim, (static_cast<int>(blockIdx.x) + 1) * c.span);
  for (int first_col = blockIdx.x * c.span; first_col < last_col; first_col += MAX_SLICE) {
    const int cols = min(MAX_SLICE, a.vdim - first_col);
    __syncthreads();
    if (wide) {
      for (int i = t; i < dim4 * (MAX_SLICE / 4); i += THREADS) {
        const int r = i / (MAX_SLICE / 4), e = (i - r * (MAX_SLICE / 4)) * 4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r < a.dim && e < cols) v = *reinterpret_cast<const float4*>(before + static_cast<size_t>(r) * a.vdim + first_col + e);
        *reinterpret_cast<float4*>(s_s + r * MAX_SLICE + e) = v;
      }
    } else {
      for (int i = t; i < dim4 * MAX_SLICE; i += THREADS) {
        const int r = i / MAX_SLICE, e = i - r * MAX_SLICE;
        s_s[i] = (r < a.dim && e < cols) ? before[static_cast<size_t>(r) * a.vdim + first_col + e] : 0.f;
      }
    }
    __syncthreads();
    float acc[4][4] = {};
    for (int e = 0; e < dim4; e += 4) {
      float4 sv[4];
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) sv[kk] = *reinterpret_cast<const float4*>(s_s + (e + kk) * MAX_SLICE + 4 * tx);
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const float4 q = *reinterpret_cast<const float4*>(q_s + (ty + 16 * r) * pitch + e);
        fma4(acc[r], q.x, sv[0]); fma4(acc[r], q.y, sv[1]); fma4(acc[r], q.z, sv[2]); fma4(acc[r], q.w, sv[3]);
      }
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int qi = ty + 16 * r;
      if (qi >= count) continue;
      const float p = pow_s[qi + 1];
      float* o = a.out + static_cast<size_t>(first + qi) * out_pitch + head * a.vdim + first_col + 4 * tx;
      if (wide) {
        if (4 * tx < cols) {
          float4 v = *reinterpret_cast<float4*>(o);
          v.x = fmaf(p, acc[r][0], v.x); v.y = fmaf(p, acc[r][1], v.y); v.z = fmaf(p, acc[r][2], v.z); v.w = fmaf(p, acc[r][3], v.w);
          *reinterpret_cast<float4*>(o) = v;
        }
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (4 * tx + e < cols) o[e] = fmaf(p, acc[r][e], o[e]);
      }
    }
  }
}

// ---- norm_gate ------------------------------------------------------------------------------------------------
// grid (rows, parts): a row's columns are shared among `parts` blocks (few rows fill the device all the same); with
// a weight every block forms the row's sum of squares itself, in the same order.
// VEC = 4: 16-byte accesses (the width, the gate's first column and the fused row's width multiples of four).
template <typename T, int VEC>
__global__ void __launch_bounds__(THREADS) norm_gate_kernel(const float* __restrict__ x, const float* __restrict__ gates,
                                                            int partials, long long partial_stride, int row_width, int gate_at,
                                                            const float* __restrict__ weight, float eps, T* __restrict__ out,
                                                            int width) {
  __shared__ float scratch[33];
  let_dependents_start();
  wait_for_previous();
  const int row = blockIdx.x, groups = width / VEC;
  const float* src = x + static_cast<size_t>(row) * width;
  float gain = 1.0f;
  if (weight != nullptr) {
    float sq = 0.f;
    for (int g = threadIdx.x; g < groups; g += THREADS) {
      float v[VEC];
      if constexpr (VEC == 4) load4<float>(src + g * 4, v);
      else v[0] = src[g];
#pragma unroll
      for (int e = 0; e < VEC; ++e) sq = fmaf(v[e], v[e], sq);
    }
    gain = 1.0f / sqrtf(block_sum(sq, scratch) / static_cast<float>(width) + eps);
  }
  const int each = (groups + gridDim.y - 1) / gridDim.y;
  const int begin = blockIdx.y * each, end = min(groups, begin + each);
  for (int g = begin + threadIdx.x; g < end; g += THREADS) {
    const int i = g * VEC;
    float v[VEC], w[VEC], gate[VEC];
    if constexpr (VEC == 4) {
      load4<float>(src + i, v);
      if (weight != nullptr) load4<float>(weight + i, w);
      if (gates != nullptr) sum_partials4(gates + static_cast<size_t>(row) * row_width + gate_at + i, partial_stride, partials, gate);
    } else {
      v[0] = src[i];
      if (weight != nullptr) w[0] = weight[i];
      if (gates != nullptr) gate[0] = sum_partials(gates + static_cast<size_t>(row) * row_width + gate_at + i, partial_stride, partials);
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      if (weight != nullptr) v[e] = v[e] * gain * w[e];
      if (gates != nullptr) v[e] = v[e] / (1.0f + expf(-gate[e]));
    }
    T* dst = out + static_cast<size_t>(row) * width + i;
    if constexpr (VEC == 4) store4<T>(dst, v);
    else dst[0] = from_float<T>(v[0]);
  }
}

// ---- latent_rope_store ------------------------------------------------------------------------------------------
// fused row: heads x [rank | rot] queries, then [rank | rot] of the token itself.  Inside a rotated part, dimension i
// pairs with i + rot/2 and turns by position * inv_freq[i]; cos and sin are multiplied by `gain`.
// grid (tokens, parts): the token's units (query head 0 .. heads - 1, then its own page row) are shared among
// `parts` blocks, unit blockIdx.y, blockIdx.y + parts, ...  The rotation's sines and cosines depend on the token
// alone: a block forms them once.
template <typename T>
__global__ void __launch_bounds__(THREADS) latent_rope_store_kernel(
    const float* __restrict__ fused, int partials, long long partial_stride, int row_width, const float* __restrict__ latent_weight,
    float eps, const int* __restrict__ positions, const float* __restrict__ inv_freq, float gain, T* __restrict__ q_out,
    T* __restrict__ cache, const int* __restrict__ slots, int heads, int rank, int rot, int padded, long long num_slots) {
  extern __shared__ __align__(16) float latent[];   // [rank], then cos and sin times the gain [rot / 2] each
  __shared__ float scratch[33];
  let_dependents_start();
  wait_for_previous();
  const int token = blockIdx.x, half = rot / 2, each = rank + rot;
  float* cos_s = latent + rank;
  float* sin_s = cos_s + half;
  const float* row = fused + static_cast<size_t>(token) * row_width;
  const float position = static_cast<float>(positions[token]);
  for (int i = threadIdx.x; i < half; i += THREADS) {
    float sn, cs;
    sincosf(position * inv_freq[i], &sn, &cs);
    cos_s[i] = cs * gain;
    sin_s[i] = sn * gain;
  }
  __syncthreads();
  for (int unit = blockIdx.y; unit <= heads; unit += gridDim.y) {
    const float* own = row + unit * each;
    if (unit < heads) {   // a query head: the latent-space part is cast, the rotated part turned
      T* dst = q_out + (static_cast<size_t>(token) * heads + unit) * padded;
      for (int e = threadIdx.x; e < padded; e += THREADS) {
        float v = 0.f;
        if (e < rank) {
          v = sum_partials(own + e, partial_stride, partials);
        } else if (e < each) {
          const int r = e - rank, pair = r < half ? r : r - half;
          const float lo = sum_partials(own + rank + pair, partial_stride, partials);
          const float hi = sum_partials(own + rank + pair + half, partial_stride, partials);
          v = r < half ? lo * cos_s[pair] - hi * sin_s[pair] : hi * cos_s[pair] + lo * sin_s[pair];
        }
        dst[e] = from_float<T>(v);
      }
      continue;
    }
    if (cache == nullptr) return;
    long long slot = slots[token];
    if (slot < 0 || slot >= num_slots) slot = -1;
    float sq = 0.f;
    for (int i = threadIdx.x; i < rank; i += THREADS) {
      const float v = sum_partials(own + i, partial_stride, partials);
      latent[i] = v;
      sq = fmaf(v, v, sq);
    }
    const float unit_gain = 1.0f / sqrtf(block_sum(sq, scratch) / static_cast<float>(rank) + eps);
    if (slot < 0) return;
    T* dst = cache + static_cast<size_t>(slot) * padded;
    for (int e = threadIdx.x; e < padded; e += THREADS) {
      float v = 0.f;
      if (e < rank) {
        v = latent[e] * unit_gain * latent_weight[e];
      } else if (e < each) {
        const int r = e - rank, pair = r < half ? r : r - half;
        const float lo = sum_partials(own + rank + pair, partial_stride, partials);
        const float hi = sum_partials(own + rank + pair + half, partial_stride, partials);
        v = r < half ? lo * cos_s[pair] - hi * sin_s[pair] : hi * cos_s[pair] + lo * sin_s[pair];
      }
      dst[e] = from_float<T>(v);
    }
  }
}

// ---- concat_cast ------------------------------------------------------------------------------------------------
struct Terms {
  const float* data[4];
  int partials[4];
  long long stride[4];
  float scale[4];
  int count;
};

template <typename T>
__global__ void __launch_bounds__(THREADS) concat_cast_kernel(float* __restrict__ resid, Terms terms, const float* __restrict__ other,
                                                              T* __restrict__ out, long long total, int width) {
  let_dependents_start();
  wait_for_previous();
  const long long i = static_cast<long long>(blockIdx.x) * THREADS + threadIdx.x;
  if (i >= total) return;
  const long long row = i / width;
  const int e = static_cast<int>(i - row * width);
  float v = resid[i];
  if (terms.count > 0) {
    for (int k = 0; k < terms.count; ++k)
      v = fmaf(terms.scale[k], sum_partials(terms.data[k] + i, terms.stride[k], terms.partials[k]), v);
    resid[i] = v;
  }
  out[row * 2 * width + e] = from_float<T>(v);
  out[row * 2 * width + width + e] = from_float<T>(other[i]);
}

}  // namespace decay

// Blocks a row of work is shared among, at most `most`: few rows are spread until the blocks fill the device twice.
static int shrike_spread(int rows, int most) {
  const int wanted = (2 * shrike_device().sm_count + rows - 1) / rows;
  return wanted < 1 ? 1 : (wanted > most ? most : wanted);
}

// Runs of CHUNK tokens a batch of `n` tokens in `seqs` sequences makes at most.
SHRIKE_API long long shrike_decay_scan_chunks(int n, int seqs) { return n / decay::CHUNK + seqs; }
SHRIKE_API int shrike_decay_scan_chunk() { return decay::CHUNK; }

// `longest`: the most new tokens a sequence of the batch brings, `n` the batch's tokens.  With `chunk_from` > 0 and
// `longest` >= `chunk_from`, sequences that bring at least `chunk_from` tokens run in the chunked form, for which the
// caller holds `chunk_state` (float32, shrike_decay_scan_chunks(n, seqs) * heads * dim * vdim); the others walk.
SHRIKE_API int shrike_decay_scan(const float* fused, int partials, long long partial_stride, int row_width, const float* decays,
                                 float* state, const int* q_start, const int* state_slot, float* out, int num_seqs, int heads,
                                 int dim, int vdim, int num_slots, int state_stride, int longest, int chunk_from, int n,
                                 float* chunk_state, cudaStream_t stream) {
  using namespace decay;
  if (num_seqs <= 0) return SHRIKE_OK;
  if (heads <= 0 || dim <= 0 || vdim <= 0 || state_stride < dim * vdim || partials < 1) return SHRIKE_BAD_ARGUMENT;
  ScanArgs a;
  a.fused = fused; a.partials = partials; a.partial_stride = partial_stride; a.row_width = row_width; a.decays = decays;
  a.state = state; a.q_start = q_start; a.state_slot = state_slot; a.out = out;
  a.heads = heads; a.dim = dim; a.vdim = vdim; a.num_slots = num_slots; a.state_stride = state_stride;
  a.slice = vdim < MAX_SLICE ? vdim : MAX_SLICE;
  a.groups = THREADS / a.slice;
  if (a.groups > dim) a.groups = dim;
  const int slices = (vdim + a.slice - 1) / a.slice;
  const int rows = (dim + a.groups - 1) / a.groups;
  // runs of tokens only where their shared memory fits; a head too tall for the walk's registers walks through memory
  const size_t pitch = chunk_pitch(dim), dim4 = (static_cast<size_t>(dim) + 3) & ~static_cast<size_t>(3);
  const size_t local_smem = (2 * CHUNK * pitch + static_cast<size_t>(CHUNK) * MAX_SLICE + CHUNK * SCORE_PITCH + CHUNK + 4) * sizeof(float);
  const size_t finish_smem = (CHUNK * pitch + dim4 * MAX_SLICE + CHUNK + 4) * sizeof(float);
  const size_t limit = shrike_device().max_smem;
  const bool chunked = chunk_state != nullptr && chunk_from > 0 && longest >= chunk_from && local_smem <= limit && finish_smem <= limit;
  const int chunks = static_cast<int>(shrike_decay_scan_chunks(n, num_seqs));
  const int skip = chunked ? chunk_from - 1 : 0;
  const dim3 grid(slices, heads, num_seqs);
  const size_t smem = (2 * static_cast<size_t>(dim) + a.slice + static_cast<size_t>(a.groups) * a.slice) * sizeof(float);
  if (smem > 48 * 1024) return SHRIKE_BAD_ARGUMENT;
  cudaError_t err;
#define SHRIKE_WALK(R) err = launch_dependent(walk_kernel<R>, grid, dim3(THREADS), smem, stream, a, skip)
  if (rows > 64) err = launch_dependent(walk_in_memory_kernel, grid, dim3(THREADS), smem, stream, a, skip);
  else if (rows <= 8) SHRIKE_WALK(8);
  else if (rows <= 16) SHRIKE_WALK(16);
  else if (rows <= 32) SHRIKE_WALK(32);
  else SHRIKE_WALK(64);
#undef SHRIKE_WALK
  if (err != cudaSuccess) return static_cast<int>(err);
  if (chunked) {
    ChunkArgs c;
    c.s = a; c.chunk_state = chunk_state; c.num_seqs = num_seqs; c.skip = skip;
    static size_t raised_local = 0, raised_finish = 0;
    if (local_smem > raised_local) {
      if (cudaFuncSetAttribute(chunk_local_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(limit)) != cudaSuccess)
        return SHRIKE_BAD_ARGUMENT;
      raised_local = limit;
    }
    if (finish_smem > raised_finish) {
      if (cudaFuncSetAttribute(chunk_finish_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(limit)) != cudaSuccess)
        return SHRIKE_BAD_ARGUMENT;
      raised_finish = limit;
    }
    // a CTA takes every value column of its run and head (q, k and the scores are staged once) when the runs and heads
    // alone fill the device twice over, else 64 columns
    c.span = static_cast<long long>(chunks) * heads >= 2ll * shrike_device().sm_count ? slices * MAX_SLICE : MAX_SLICE;
    const dim3 per_chunk((vdim + c.span - 1) / c.span, heads, chunks);
    err = launch_dependent(chunk_local_kernel, per_chunk, dim3(THREADS), local_smem, stream, c);
    if (err != cudaSuccess) return static_cast<int>(err);
    // four elements a thread where every head's state and every run's addition start on 16 bytes
    const bool carry_wide = (dim * vdim) % 4 == 0 && state_stride % 4 == 0;
    const int carry_threads = carry_wide ? dim * vdim / 4 : dim * vdim;
    const dim3 per_seq((carry_threads + THREADS - 1) / THREADS, heads, num_seqs);
    err = carry_wide ? launch_dependent(chunk_carry_kernel<4>, per_seq, dim3(THREADS), 0, stream, c)
                     : launch_dependent(chunk_carry_kernel<1>, per_seq, dim3(THREADS), 0, stream, c);
    if (err != cudaSuccess) return static_cast<int>(err);
    err = launch_dependent(chunk_finish_kernel, per_chunk, dim3(THREADS), finish_smem, stream, c);
    if (err != cudaSuccess) return static_cast<int>(err);
  }
  return shrike_launch_status();
}

SHRIKE_API int shrike_norm_gate(const float* x, const float* gates, int partials, long long partial_stride, int row_width,
                                int gate_at, const float* weight, float eps, void* out, int dtype, int n, int width,
                                cudaStream_t stream) {
  if (n <= 0) return SHRIKE_OK;
  if (width <= 0) return SHRIKE_BAD_ARGUMENT;
  const auto on16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  const bool wide = width % 4 == 0 && on16(x) && on16(out) && on16(weight) &&
                    (gates == nullptr || (on16(gates) && gate_at % 4 == 0 && row_width % 4 == 0 && partial_stride % 4 == 0));
  const int parts = shrike_spread(n, ((wide ? width / 4 : width) + decay::THREADS - 1) / decay::THREADS);
#define SHRIKE_NORM_GATE(T)                                                                                                \
  (wide ? launch_dependent(decay::norm_gate_kernel<T, 4>, dim3(n, parts), dim3(decay::THREADS), 0, stream, x, gates, partials, \
                           partial_stride, row_width, gate_at, weight, eps, static_cast<T*>(out), width)                     \
        : launch_dependent(decay::norm_gate_kernel<T, 1>, dim3(n, parts), dim3(decay::THREADS), 0, stream, x, gates, partials, \
                           partial_stride, row_width, gate_at, weight, eps, static_cast<T*>(out), width))
  if (dtype == SHRIKE_F32) SHRIKE_NORM_GATE(float);
  else if (dtype == SHRIKE_BF16) SHRIKE_NORM_GATE(__nv_bfloat16);
  else return SHRIKE_BAD_ARGUMENT;
#undef SHRIKE_NORM_GATE
  return shrike_launch_status();
}

SHRIKE_API int shrike_latent_rope_store(const float* fused, int partials, long long partial_stride, int row_width,
                                        const float* latent_weight, float eps, const int* positions, const float* inv_freq,
                                        float gain, void* q_out, void* cache, const int* slots, int dtype, int n, int heads,
                                        int rank, int rot, int padded, long long num_slots, cudaStream_t stream) {
  if (n <= 0) return SHRIKE_OK;
  if (heads <= 0 || rank <= 0 || rot < 2 || rot % 2 || padded < rank + rot) return SHRIKE_BAD_ARGUMENT;
  const size_t smem = static_cast<size_t>(rank + rot) * sizeof(float);
  const int parts = shrike_spread(n, heads + 1);
#define SHRIKE_LATENT_ROPE(T)                                                                                          \
  launch_dependent(decay::latent_rope_store_kernel<T>, dim3(n, parts), dim3(decay::THREADS), smem, stream, fused, partials, \
                   partial_stride, row_width, latent_weight, eps, positions, inv_freq, gain, static_cast<T*>(q_out),     \
                   static_cast<T*>(cache), slots, heads, rank, rot, padded, num_slots)
  if (dtype == SHRIKE_F32) SHRIKE_LATENT_ROPE(float);
  else if (dtype == SHRIKE_BF16) SHRIKE_LATENT_ROPE(__nv_bfloat16);
  else return SHRIKE_BAD_ARGUMENT;
#undef SHRIKE_LATENT_ROPE
  return shrike_launch_status();
}

// terms: up to four pending sums (data, partials, stride in elements, scale), added to `resid` in order.
SHRIKE_API int shrike_concat_cast(float* resid, const float* const* data, const int* partials, const long long* strides,
                                  const float* scales, int count, const float* other, void* out, int dtype, int n, int width,
                                  cudaStream_t stream) {
  if (n <= 0) return SHRIKE_OK;
  if (count < 0 || count > 4 || width <= 0) return SHRIKE_BAD_ARGUMENT;
  decay::Terms terms;
  terms.count = count;
  for (int k = 0; k < 4; ++k) {
    terms.data[k] = k < count ? data[k] : nullptr;
    terms.partials[k] = k < count ? partials[k] : 1;
    terms.stride[k] = k < count ? strides[k] : 0;
    terms.scale[k] = k < count ? scales[k] : 0.f;
  }
  const long long total = static_cast<long long>(n) * width;
  const long long blocks = (total + decay::THREADS - 1) / decay::THREADS;
  if (blocks > 0x7fffffffLL) return SHRIKE_BAD_ARGUMENT;
#define SHRIKE_CONCAT(T)                                                                                        \
  launch_dependent(decay::concat_cast_kernel<T>, dim3(static_cast<unsigned>(blocks)), dim3(decay::THREADS), 0, stream, resid, \
                   terms, other, static_cast<T*>(out), total, width)
  if (dtype == SHRIKE_F32) SHRIKE_CONCAT(float);
  else if (dtype == SHRIKE_BF16) SHRIKE_CONCAT(__nv_bfloat16);
  else return SHRIKE_BAD_ARGUMENT;
#undef SHRIKE_CONCAT
  return shrike_launch_status();
}
