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

// grid (vdim slices, heads, chunks): intra-run outputs and L_c for a slice of columns.
__global__ void __launch_bounds__(THREADS) chunk_local_kernel(ChunkArgs c) {
  extern __shared__ __align__(16) float shared[];
  const ScanArgs& a = c.s;
  float* q_s = shared;                              // [CHUNK][dim + 1]
  float* k_s = q_s + CHUNK * (a.dim + 1);           // [CHUNK][dim + 1]
  float* v_s = k_s + CHUNK * (a.dim + 1);           // [CHUNK][slice]
  float* w_s = v_s + CHUNK * a.slice;               // [CHUNK][CHUNK + 1] decayed scores
  let_dependents_start();
  wait_for_previous();
  const int run = blockIdx.z, head = blockIdx.y, first_col = blockIdx.x * a.slice;
  int seq, first, count;
  if (!locate_run(c, run, seq, first, count)) return;
  const int slot = a.state_slot[seq];
  if (slot < 0 || slot >= a.num_slots) return;
  const int cols = min(a.slice, a.vdim - first_col);
  const int t = threadIdx.x, pitch = a.dim + 1;
  const float d = a.decays[head];
  const int q_at = head * a.dim, k_at = a.heads * a.dim + head * a.dim, v_at = 2 * a.heads * a.dim + head * a.vdim + first_col;
  for (int i = t; i < count * a.dim; i += THREADS) {
    const int j = i / a.dim, e = i - j * a.dim;
    const float* row = a.fused + static_cast<size_t>(first + j) * a.row_width;
    q_s[j * pitch + e] = silu(sum_partials(row + q_at + e, a.partial_stride, a.partials));
    k_s[j * pitch + e] = silu(sum_partials(row + k_at + e, a.partial_stride, a.partials));
  }
  for (int i = t; i < count * cols; i += THREADS) {
    const int j = i / cols, e = i - j * cols;
    const float* row = a.fused + static_cast<size_t>(first + j) * a.row_width;
    v_s[j * a.slice + e] = silu(sum_partials(row + v_at + e, a.partial_stride, a.partials));
  }
  __syncthreads();
  // decayed scores w[i][j] = d^(i - j) q_i . k_j for j <= i
  for (int i = t; i < count * count; i += THREADS) {
    const int qi = i / count, kj = i - qi * count;
    float dot = 0.f;
    if (kj <= qi) {
      for (int e = 0; e < a.dim; ++e) dot = fmaf(q_s[qi * pitch + e], k_s[kj * pitch + e], dot);
      dot *= int_power(d, qi - kj);
    }
    w_s[qi * (CHUNK + 1) + kj] = dot;
  }
  __syncthreads();
  for (int i = t; i < count * cols; i += THREADS) {
    const int qi = i / cols, e = i - qi * cols;
    float sum = 0.f;
    for (int kj = 0; kj <= qi; ++kj) sum = fmaf(w_s[qi * (CHUNK + 1) + kj], v_s[kj * a.slice + e], sum);
    a.out[static_cast<size_t>(first + qi) * a.heads * a.vdim + head * a.vdim + first_col + e] = sum;
  }
  // L_c[r][e] = sum_j d^(count - 1 - j) k_j[r] v_j[e]; the powers go into w_s's first row
  __syncthreads();
  for (int j = t; j < count; j += THREADS) w_s[j] = int_power(d, count - 1 - j);
  __syncthreads();
  float* local = c.chunk_state + (static_cast<size_t>(run) * a.heads + head) * a.dim * a.vdim;
  for (int i = t; i < a.dim * cols; i += THREADS) {
    const int r = i / cols, e = i - r * cols;
    float sum = 0.f;
    for (int j = 0; j < count; ++j) sum = fmaf(w_s[j] * k_s[j * pitch + r], v_s[j * a.slice + e], sum);
    local[static_cast<size_t>(r) * a.vdim + first_col + e] = sum;
  }
}

// grid (blocks over dim * vdim, heads, seqs): walks a sequence's runs in order, element by element.
__global__ void __launch_bounds__(THREADS) chunk_carry_kernel(ChunkArgs c) {
  const ScanArgs& a = c.s;
  let_dependents_start();
  wait_for_previous();
  const int seq = blockIdx.z, head = blockIdx.y;
  const int slot = a.state_slot[seq];
  if (slot < 0 || slot >= a.num_slots) return;
  const int length = a.q_start[seq + 1] - a.q_start[seq];
  if (length <= c.skip) return;   // the walk serves it
  const int element = blockIdx.x * THREADS + threadIdx.x;
  if (element >= a.dim * a.vdim) return;
  int run = 0;   // the sequence's first run: those of the sequences before it come first
  for (int s = 0; s < seq; ++s) {
    const int other = a.q_start[s + 1] - a.q_start[s];
    if (other > c.skip) run += (other + CHUNK - 1) / CHUNK;
  }
  const float d = a.decays[head];
  float* mine = a.state + (static_cast<size_t>(slot) * a.heads + head) * a.state_stride + element;
  float held = *mine;
  for (int done = 0; done < length; done += CHUNK, ++run) {
    float* local = c.chunk_state + (static_cast<size_t>(run) * a.heads + head) * a.dim * a.vdim + element;
    const float add = *local;
    *local = held;                                   // S before this run: what `finish` reads
    held = fmaf(int_power(d, min(CHUNK, length - done)), held, add);
  }
  *mine = held;
}

// grid (vdim slices, heads, chunks): o_t += d^(t - a + 1) S_before^T q_t.
__global__ void __launch_bounds__(THREADS) chunk_finish_kernel(ChunkArgs c) {
  extern __shared__ __align__(16) float shared[];
  const ScanArgs& a = c.s;
  float* q_s = shared;                        // [CHUNK][dim + 1]
  float* s_s = q_s + CHUNK * (a.dim + 1);     // [dim][slice]
  let_dependents_start();
  wait_for_previous();
  const int run = blockIdx.z, head = blockIdx.y, first_col = blockIdx.x * a.slice;
  int seq, first, count;
  if (!locate_run(c, run, seq, first, count)) return;
  const int slot = a.state_slot[seq];
  if (slot < 0 || slot >= a.num_slots) return;
  const int cols = min(a.slice, a.vdim - first_col);
  const int t = threadIdx.x, pitch = a.dim + 1;
  const float d = a.decays[head];
  const int q_at = head * a.dim;
  for (int i = t; i < count * a.dim; i += THREADS) {
    const int j = i / a.dim, e = i - j * a.dim;
    const float* row = a.fused + static_cast<size_t>(first + j) * a.row_width;
    q_s[j * pitch + e] = silu(sum_partials(row + q_at + e, a.partial_stride, a.partials));
  }
  const float* before = c.chunk_state + (static_cast<size_t>(run) * a.heads + head) * a.dim * a.vdim;
  for (int i = t; i < a.dim * cols; i += THREADS) {
    const int r = i / cols, e = i - r * cols;
    s_s[r * a.slice + e] = before[static_cast<size_t>(r) * a.vdim + first_col + e];
  }
  __syncthreads();
  for (int i = t; i < count * cols; i += THREADS) {
    const int qi = i / cols, e = i - qi * cols;
    float sum = 0.f;
    for (int r = 0; r < a.dim; ++r) sum = fmaf(q_s[qi * pitch + r], s_s[r * a.slice + e], sum);
    float* o = a.out + static_cast<size_t>(first + qi) * a.heads * a.vdim + head * a.vdim + first_col + e;
    *o = fmaf(int_power(d, qi + 1), sum, *o);
  }
}

// ---- norm_gate ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(THREADS) norm_gate_kernel(const float* __restrict__ x, const float* __restrict__ gates,
                                                            int partials, long long partial_stride, int row_width, int gate_at,
                                                            const float* __restrict__ weight, float eps, T* __restrict__ out,
                                                            int width) {
  __shared__ float scratch[33];
  let_dependents_start();
  wait_for_previous();
  const int row = blockIdx.x;
  const float* src = x + static_cast<size_t>(row) * width;
  float gain = 1.0f;
  if (weight != nullptr) {
    float sq = 0.f;
    for (int i = threadIdx.x; i < width; i += THREADS) sq = fmaf(src[i], src[i], sq);
    gain = 1.0f / sqrtf(block_sum(sq, scratch) / static_cast<float>(width) + eps);
  }
  for (int i = threadIdx.x; i < width; i += THREADS) {
    float v = src[i];
    if (weight != nullptr) v = v * gain * weight[i];
    if (gates != nullptr) {
      const float g = sum_partials(gates + static_cast<size_t>(row) * row_width + gate_at + i, partial_stride, partials);
      v = v / (1.0f + expf(-g));
    }
    out[static_cast<size_t>(row) * width + i] = from_float<T>(v);
  }
}

// ---- latent_rope_store ------------------------------------------------------------------------------------------
// fused row: heads x [rank | rot] queries, then [rank | rot] of the token itself.  Inside a rotated part, dimension i
// pairs with i + rot/2 and turns by position * inv_freq[i]; cos and sin are multiplied by `gain`.
template <typename T>
__global__ void __launch_bounds__(THREADS) latent_rope_store_kernel(
    const float* __restrict__ fused, int partials, long long partial_stride, int row_width, const float* __restrict__ latent_weight,
    float eps, const int* __restrict__ positions, const float* __restrict__ inv_freq, float gain, T* __restrict__ q_out,
    T* __restrict__ cache, const int* __restrict__ slots, int heads, int rank, int rot, int padded, long long num_slots) {
  extern __shared__ __align__(16) float latent[];   // [rank]
  __shared__ float scratch[33];
  let_dependents_start();
  wait_for_previous();
  const int token = blockIdx.x, half = rot / 2, each = rank + rot;
  const float* row = fused + static_cast<size_t>(token) * row_width;
  const float position = static_cast<float>(positions[token]);
  // queries: the latent-space part is cast, the rotated part turned
  for (int i = threadIdx.x; i < heads * padded; i += THREADS) {
    const int head = i / padded, e = i - head * padded;
    float v = 0.f;
    if (e < rank) {
      v = sum_partials(row + head * each + e, partial_stride, partials);
    } else if (e < each) {
      const int r = e - rank, pair = r < half ? r : r - half;
      const float angle = position * inv_freq[pair];
      float s, c;
      sincosf(angle, &s, &c);
      const float lo = sum_partials(row + head * each + rank + pair, partial_stride, partials);
      const float hi = sum_partials(row + head * each + rank + pair + half, partial_stride, partials);
      v = r < half ? (lo * c - hi * s) * gain : (hi * c + lo * s) * gain;
    }
    q_out[static_cast<size_t>(token) * heads * padded + i] = from_float<T>(v);
  }
  if (cache == nullptr) return;
  long long slot = slots[token];
  if (slot < 0 || slot >= num_slots) slot = -1;
  const float* own = row + heads * each;
  float sq = 0.f;
  for (int i = threadIdx.x; i < rank; i += THREADS) {
    const float v = sum_partials(own + i, partial_stride, partials);
    latent[i] = v;
    sq = fmaf(v, v, sq);
  }
  const float unit = 1.0f / sqrtf(block_sum(sq, scratch) / static_cast<float>(rank) + eps);
  if (slot < 0) return;
  T* dst = cache + static_cast<size_t>(slot) * padded;
  for (int e = threadIdx.x; e < padded; e += THREADS) {
    float v = 0.f;
    if (e < rank) {
      v = latent[e] * unit * latent_weight[e];
    } else if (e < each) {
      const int r = e - rank, pair = r < half ? r : r - half;
      const float angle = position * inv_freq[pair];
      float s, c;
      sincosf(angle, &s, &c);
      const float lo = sum_partials(own + rank + pair, partial_stride, partials);
      const float hi = sum_partials(own + rank + pair + half, partial_stride, partials);
      v = r < half ? (lo * c - hi * s) * gain : (hi * c + lo * s) * gain;
    }
    dst[e] = from_float<T>(v);
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
  if (rows > 64) return SHRIKE_BAD_ARGUMENT;
  const bool chunked = chunk_state != nullptr && chunk_from > 0 && longest >= chunk_from;
  const int chunks = static_cast<int>(shrike_decay_scan_chunks(n, num_seqs));
  const int skip = chunked ? chunk_from - 1 : 0;
  const dim3 grid(slices, heads, num_seqs);
  const size_t smem = (2 * static_cast<size_t>(dim) + a.slice + static_cast<size_t>(a.groups) * a.slice) * sizeof(float);
  cudaError_t err;
#define SHRIKE_WALK(R) err = launch_dependent(walk_kernel<R>, grid, dim3(THREADS), smem, stream, a, skip)
  if (rows <= 8) SHRIKE_WALK(8);
  else if (rows <= 16) SHRIKE_WALK(16);
  else if (rows <= 32) SHRIKE_WALK(32);
  else SHRIKE_WALK(64);
#undef SHRIKE_WALK
  if (err != cudaSuccess) return static_cast<int>(err);
  if (chunked) {
    ChunkArgs c;
    c.s = a; c.chunk_state = chunk_state; c.num_seqs = num_seqs; c.skip = skip;
    const size_t pitch = dim + 1;
    const size_t local_smem = (2 * CHUNK * pitch + static_cast<size_t>(CHUNK) * a.slice + CHUNK * (CHUNK + 1)) * sizeof(float);
    const size_t finish_smem = (CHUNK * pitch + static_cast<size_t>(dim) * a.slice) * sizeof(float);
    const size_t limit = shrike_device().max_smem;
    if (local_smem > limit || finish_smem > limit) return SHRIKE_BAD_ARGUMENT;
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
    const dim3 per_chunk(slices, heads, chunks);
    err = launch_dependent(chunk_local_kernel, per_chunk, dim3(THREADS), local_smem, stream, c);
    if (err != cudaSuccess) return static_cast<int>(err);
    const dim3 per_seq((dim * vdim + THREADS - 1) / THREADS, heads, num_seqs);
    err = launch_dependent(chunk_carry_kernel, per_seq, dim3(THREADS), 0, stream, c);
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
#define SHRIKE_NORM_GATE(T)                                                                                              \
  launch_dependent(decay::norm_gate_kernel<T>, dim3(n), dim3(decay::THREADS), 0, stream, x, gates, partials, partial_stride, \
                   row_width, gate_at, weight, eps, static_cast<T*>(out), width)
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
  const size_t smem = static_cast<size_t>(rank) * sizeof(float);
#define SHRIKE_LATENT_ROPE(T)                                                                                          \
  launch_dependent(decay::latent_rope_store_kernel<T>, dim3(n), dim3(decay::THREADS), smem, stream, fused, partials,     \
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
