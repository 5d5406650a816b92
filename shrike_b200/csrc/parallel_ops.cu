// Kernels for layers whose branches run side by side (x += mixer(N1 x) + ff(N2 x)), for attention with
// per-head norms and a partial rotation, for a recurrent mixer with a matrix state, and for routed experts.
//
//   tanh_norm          resid += sum of pending branch outputs (each a [N, W] array or a K-split stack, each with
//                      a scale) (+ one broadcast row); then up to two norms of the same row,
//                      out_k = tanh(alpha_k x) * w_k + b_k; or the same on a few gathered rows
//   head_prep          a fused q|k|v|gate projection: bias, RMS norm per head with one weight for all heads,
//                      rotation of each head's first dimensions, q to its buffer, k and v into their pages
//                      (heads padded to the kernels' head size), sigmoid of the per-head gate
//   matrix_memory_scan the recurrence S_t = keep_t S_(t-1) + take_t k_t v_t^T of a matrix-memory mixer, token by
//                      token with the state on chip, for portions and single tokens alike
//   matrix_memory_scores / _local / _carry / _finish   the same for portions, as products over chunks of 64 tokens, every
//                      chunk on a CTA of its own
//   matrix_memory_out  its outputs: divided by their denominator, each head over its root mean square, times a
//                      weight and a sigmoid gate
//   route_top          router logits, softmax over all experts, the `top` largest renormalised, as a dense
//                      [N, experts (+ 1)] array of weights (0 where an expert is not chosen), the shared expert's
//                      sigmoid gate in the last column
//   act_mul_blocks     act(gate) * up * the weight of the column's expert
//
// Norms, gates, decays, states, routers and the residual sum are float32; a result is rounded once, when it is
// stored in the activation type.
#include "common.cuh"

namespace parallel {

constexpr int MAX_TERMS = 4;

struct SumTerm {
  const float* data;      // [partials][N][W]
  long long stride;       // elements between partials
  int partials;
  float scale;
};

struct TanhNormArgs {
  float* resid;           // [N][W]
  SumTerm terms[MAX_TERMS];
  int num_terms;
  const float* row_add;   // [W] or null: added to every row
  const int* rows;        // null: every row, the residual is rewritten; else out[r] = norm(x[rows[r]]), nothing else written
  int norms;              // 0, 1 or 2
  float alpha[2];
  const float* weight[2];
  const float* bias[2];
  void* out[2];
  int n, width;
};

// tanh in the activation type's accuracy: bfloat16 results keep 8 bits, so the hardware exponential serves
// (absolute error about 1e-7); float32 uses tanhf.
template <typename T> __device__ __forceinline__ float tanh_for(float z);
template <> __device__ __forceinline__ float tanh_for<float>(float z) { return tanhf(z); }
template <> __device__ __forceinline__ float tanh_for<__nv_bfloat16>(float z) {
  const float c = fminf(fmaxf(z, -15.f), 15.f);
  return 1.0f - __fdividef(2.0f, __expf(2.0f * c) + 1.0f);
}

template <typename TO, int VEC>
__global__ void __launch_bounds__(256) tanh_norm_kernel(const TanhNormArgs a) {
  let_dependents_start();
  wait_for_previous();
  const int groups = a.width / VEC;
  for (int row = blockIdx.y; row < a.n; row += gridDim.y) {
    const int src = a.rows != nullptr ? a.rows[row] : row;
    const size_t src_base = static_cast<size_t>(src) * a.width, out_base = static_cast<size_t>(row) * a.width;
    for (int group = blockIdx.x * blockDim.x + threadIdx.x; group < groups; group += gridDim.x * blockDim.x) {
      const int col = group * VEC;
      float x[VEC];
      if constexpr (VEC == 4) {
        load4<float>(a.resid + src_base + col, x);
        for (int t = 0; t < a.num_terms; ++t) {
          const SumTerm& term = a.terms[t];
          float part[4];
          sum_partials4(term.data + src_base + col, term.stride, term.partials, part);
#pragma unroll
          for (int e = 0; e < 4; ++e) x[e] = __fmaf_rn(term.scale, part[e], x[e]);
        }
        if (a.row_add != nullptr) {
          float part[4];
          load4<float>(a.row_add + col, part);
#pragma unroll
          for (int e = 0; e < 4; ++e) x[e] = __fadd_rn(x[e], part[e]);
        }
        if (a.rows == nullptr && (a.num_terms > 0 || a.row_add != nullptr)) store4<float>(a.resid + src_base + col, x);
      } else {
#pragma unroll
        for (int e = 0; e < VEC; ++e) x[e] = a.resid[src_base + col + e];
        for (int t = 0; t < a.num_terms; ++t) {
          const SumTerm& term = a.terms[t];
#pragma unroll
          for (int e = 0; e < VEC; ++e)
            x[e] = __fmaf_rn(term.scale, sum_partials(term.data + src_base + col + e, term.stride, term.partials), x[e]);
        }
        if (a.row_add != nullptr) {
#pragma unroll
          for (int e = 0; e < VEC; ++e) x[e] = __fadd_rn(x[e], a.row_add[col + e]);
        }
        if (a.rows == nullptr && (a.num_terms > 0 || a.row_add != nullptr)) {
#pragma unroll
          for (int e = 0; e < VEC; ++e) a.resid[src_base + col + e] = x[e];
        }
      }
      for (int k = 0; k < a.norms; ++k) {
        TO* out = static_cast<TO*>(a.out[k]) + out_base + col;
        if constexpr (VEC == 4) {
          float w[4], b[4], y[4];
          load4<float>(a.weight[k] + col, w);
          load4<float>(a.bias[k] + col, b);
#pragma unroll
          for (int e = 0; e < 4; ++e) y[e] = __fmaf_rn(tanh_for<TO>(a.alpha[k] * x[e]), w[e], b[e]);
          store4<TO>(out, y);
        } else {
#pragma unroll
          for (int e = 0; e < VEC; ++e)
            out[e] = from_float<TO>(__fmaf_rn(tanh_for<TO>(a.alpha[k] * x[e]), a.weight[k][col + e], a.bias[k][col + e]));
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------- head_prep
struct HeadPrepArgs {
  const float* fused;     // [partials][N][total]: q (H D) | k (G D) | v (G Dv) | gate (H, when gate_out)
  long long stride;
  int partials, total;
  const float* bias;      // [total] or null
  const int* positions;   // [N]
  const float* inv_freq;  // [rot / 2] or null
  int rot;                // rotated dimensions of a head (even, <= D); 0: none
  const float* q_weight;  // [D] or null
  const float* k_weight;  // [D] or null
  float eps;
  void* q_out;            // [N][H][Dp]
  void* keys;             // [slots][G][Dp] or null
  void* values;           // [slots][G][Dp]
  const int* slots;       // [N]; -1: nothing is stored
  float* gate_out;        // [N][H] or null
  int n, heads, kv_heads, dim, vdim, padded, num_slots;
  int whole_norm;         // 1: q and k are each divided by the root mean square of their WHOLE projection (all heads
                          // at once) and q_weight / k_weight hold one number a column ([H D], [G D])
  int value_norm;         // 1: every value head is divided by its own root mean square (no weight)
};

constexpr int PREP_WARPS = 4;

template <typename T>
__device__ __forceinline__ void head_prep_unit(const HeadPrepArgs& a, const float* row, int token, int unit, float* mine,
                                               const float* cosines, const float* sines, int lane, const float* whole) {
  const int q_cols = a.heads * a.dim, k_cols = a.kv_heads * a.dim, v_cols = a.kv_heads * a.vdim;
  if (unit == a.heads + 2 * a.kv_heads) {   // the gates: one number a head
    for (int h = lane; h < a.heads; h += 32) {
      const int col = q_cols + k_cols + v_cols + h;
      float z = sum_partials(row + col, a.stride, a.partials);
      if (a.bias != nullptr) z = __fadd_rn(z, a.bias[col]);
      a.gate_out[static_cast<size_t>(token) * a.heads + h] = 1.0f / (1.0f + expf(-z));
    }
    return;
  }
  const bool is_q = unit < a.heads, is_k = !is_q && unit < a.heads + a.kv_heads;
  const int head = is_q ? unit : (is_k ? unit - a.heads : unit - a.heads - a.kv_heads);
  const int size = (is_q || is_k) ? a.dim : a.vdim;
  const int first_col = is_q ? head * a.dim : (is_k ? q_cols + head * a.dim : q_cols + k_cols + head * a.vdim);
  const int slot = a.slots[token];
  T* dst;
  if (is_q) dst = static_cast<T*>(a.q_out) + (static_cast<size_t>(token) * a.heads + head) * a.padded;
  else {
    if (a.keys == nullptr || slot < 0 || slot >= a.num_slots) return;
    dst = static_cast<T*>(is_k ? a.keys : a.values) + (static_cast<size_t>(slot) * a.kv_heads + head) * a.padded;
  }
  const float* weight = is_q ? a.q_weight : (is_k ? a.k_weight : nullptr);
  if (a.whole_norm && weight != nullptr) weight += head * a.dim;
  const bool normed = weight != nullptr || (!is_q && !is_k && a.value_norm);
  const int half = (is_q || is_k) && a.inv_freq != nullptr ? a.rot / 2 : 0;
  // four consecutive elements a lane, 16-byte accesses, where sizes and addresses allow
  const bool wide = (size & 3) == 0 && (a.padded & 3) == 0 && (first_col & 3) == 0 && (a.total & 3) == 0 && (a.stride & 3) == 0 &&
                    (half & 3) == 0 && (reinterpret_cast<uintptr_t>(a.fused) & 15) == 0 &&
                    (reinterpret_cast<uintptr_t>(a.bias) & 15) == 0 && (reinterpret_cast<uintptr_t>(weight) & 15) == 0 &&
                    (reinterpret_cast<uintptr_t>(dst) & 15) == 0;
  float squares = 0.f;
  if (wide) {
    for (int d = lane * 4; d < size; d += 128) {
      float v[4];
      sum_partials4(row + first_col + d, a.stride, a.partials, v);
      if (a.bias != nullptr) {
        float b[4];
        load4<float>(a.bias + first_col + d, b);
#pragma unroll
        for (int e = 0; e < 4; ++e) v[e] = __fadd_rn(v[e], b[e]);
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        mine[d + e] = v[e];
        squares = __fmaf_rn(v[e], v[e], squares);
      }
    }
    if (normed) {
      const float r = a.whole_norm && weight != nullptr ? whole[is_q ? 0 : 1]
                                                        : rsqrtf(warp_sum(squares) / static_cast<float>(size) + a.eps);
      for (int d = lane * 4; d < size; d += 128) {
        float w[4] = {1.f, 1.f, 1.f, 1.f};
        if (weight != nullptr) load4<float>(weight + d, w);
#pragma unroll
        for (int e = 0; e < 4; ++e) mine[d + e] = mine[d + e] * r * w[e];
      }
    }
    __syncwarp();
    for (int d = lane * 4; d < a.padded; d += 128) {
      float v[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int at = d + e;
        v[e] = at < size ? mine[at] : 0.f;
        if (at < 2 * half) {
          const int i = at < half ? at : at - half;
          const float sine = sines[i], cosine = cosines[i];
          const float u = mine[i], w = mine[i + half];
          v[e] = at < half ? __fsub_rn(__fmul_rn(u, cosine), __fmul_rn(w, sine)) : __fadd_rn(__fmul_rn(w, cosine), __fmul_rn(u, sine));
        }
      }
      store4<T>(dst + d, v);
    }
    return;
  }
  for (int d = lane; d < size; d += 32) {
    float v = sum_partials(row + first_col + d, a.stride, a.partials);
    if (a.bias != nullptr) v = __fadd_rn(v, a.bias[first_col + d]);
    mine[d] = v;
    squares = __fmaf_rn(v, v, squares);
  }
  if (normed) {
    const float r = a.whole_norm && weight != nullptr ? whole[is_q ? 0 : 1]
                                                      : rsqrtf(warp_sum(squares) / static_cast<float>(size) + a.eps);
    for (int d = lane; d < size; d += 32) mine[d] = mine[d] * r * (weight != nullptr ? weight[d] : 1.f);
  }
  __syncwarp();
  for (int d = lane; d < a.padded; d += 32) {
    float v = d < size ? mine[d] : 0.f;
    if (d < 2 * half) {
      const int i = d < half ? d : d - half;
      const float sine = sines[i], cosine = cosines[i];
      const float u = mine[i], w = mine[i + half];
      v = d < half ? __fsub_rn(__fmul_rn(u, cosine), __fmul_rn(w, sine)) : __fadd_rn(__fmul_rn(w, cosine), __fmul_rn(u, sine));
    }
    dst[d] = from_float<T>(v);
  }
}

// A block serves one token's units (query heads, key heads, value heads, the gates) numbered blockIdx.y, blockIdx.y +
// gridDim.y, ...: few tokens are spread over many blocks, many tokens get one block each.  The rotation's sines and
// cosines depend on the token alone: the block forms them once and every head uses them.
template <typename T>
__global__ void __launch_bounds__(PREP_WARPS * 32) head_prep_kernel(const HeadPrepArgs a) {
  extern __shared__ float prep_shared[];   // [PREP_WARPS][padded] a warp's head, then [rot / 2] cosines and sines
  let_dependents_start();
  wait_for_previous();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int units = a.heads + 2 * a.kv_heads + (a.gate_out != nullptr ? 1 : 0);
  const int token = blockIdx.x;
  const float* row = a.fused + static_cast<size_t>(token) * a.total;
  const int table_half = a.inv_freq != nullptr ? a.rot / 2 : 0;
  float* cosines = prep_shared + static_cast<size_t>(PREP_WARPS) * a.padded;
  float* sines = cosines + table_half;
  const float position = static_cast<float>(a.positions[token]);
  for (int i = threadIdx.x; i < table_half; i += blockDim.x) sincosf(__fmul_rn(position, a.inv_freq[i]), &sines[i], &cosines[i]);
  __syncthreads();
  __shared__ float whole[2];      // whole_norm: 1 / rms of the token's whole q and k projections
  __shared__ float whole_scratch[33];
  if (a.whole_norm) {
    // every block of a token forms both statistics itself: few tokens are spread over many blocks, and the row is
    // read from the cache then
    const int q_cols = a.heads * a.dim, k_cols = a.kv_heads * a.dim;
    for (int which = 0; which < 2; ++which) {
      const int first = which == 0 ? 0 : q_cols, count = which == 0 ? q_cols : k_cols;
      const bool wanted = (which == 0 ? a.q_weight : a.k_weight) != nullptr && count > 0;
      float squares = 0.f;
      if (wanted)
        for (int c = threadIdx.x; c < count; c += blockDim.x) {
          float v = sum_partials(row + first + c, a.stride, a.partials);
          if (a.bias != nullptr) v = __fadd_rn(v, a.bias[first + c]);
          squares = __fmaf_rn(v, v, squares);
        }
      const float total = block_sum(squares, whole_scratch);
      if (threadIdx.x == 0) whole[which] = wanted ? rsqrtf(total / static_cast<float>(count) + a.eps) : 1.f;
    }
    __syncthreads();
  }
  float* mine = prep_shared + static_cast<size_t>(warp) * a.padded;
  for (int unit = blockIdx.y * PREP_WARPS + warp; unit < units; unit += gridDim.y * PREP_WARPS) {
    head_prep_unit<T>(a, row, token, unit, mine, cosines, sines, lane, whole);
    __syncwarp();   // the warp's buffer is read across lanes until a head is stored
  }
}

// ------------------------------------------------------------------------------------- matrix memory: scan
// One CTA owns `cols` value columns of one head's state for one sequence and walks the sequence's new tokens in
// order.  Thread j holds column j: S[:, j] lives in shared memory as S[d * ld + j].  The normaliser z (the
// recurrence with v = 1) is one more column, kept by the CTA of the head's first columns.  Tokens are staged
// TOKENS at a time (q, k, this CTA's v columns, the two gates), so the walk itself touches shared memory only.
// The state of a slot: per head `head_stride` floats (a multiple of four, so that every head starts on 16 bytes):
// D * Dv of S (row d, column j at d * Dv + j), D of z, then m.
struct ScanArgs {
  const float* fused;     // [partials][N][total]: q (H D) | k (H D) | v (H Dv) | gate (H Dv) | i (H) | f (H)
  long long stride;
  int partials, total;
  const float* gate_bias; // [2 H]: input gates, then forget gates; or null
  float* state;           // [slots][H][head_stride], head_stride >= D Dv + D + 1
  const int* q_start;     // [S + 1]
  const int* state_slot;  // [S]; -1: the sequence is padding
  float* numerator;       // [N][H][Dv]
  float* denominator;     // [N][H]
  int heads, dim, vdim, cols, num_slots;
  float cap, q_scale, floor_;
  int head_stride;
};

constexpr int SCAN_TOKENS = 8;
constexpr int SCAN_THREADS = 256;   // all of them load and store; the first cols (+ 1) walk the tokens

// A slice of a head's state matrix (rows d, columns col0 .. col0 + cols_here - 1 of [D][Dv]) between global memory
// and shared memory (row stride ld), 16 bytes at a time where the columns allow.
__device__ __forceinline__ void load_state_slice(float* S, int ld, const float* mine, int D, int Dv, int col0, int cols_here) {
  if ((Dv & 3) == 0 && (col0 & 3) == 0 && (cols_here & 3) == 0 && (reinterpret_cast<uintptr_t>(mine) & 15) == 0) {
    const int quads = cols_here >> 2;
    for (int idx = threadIdx.x; idx < D * quads; idx += blockDim.x) {
      const int d = idx / quads, j = (idx - d * quads) << 2;
      const float4 v = *reinterpret_cast<const float4*>(mine + static_cast<size_t>(d) * Dv + col0 + j);
      float* row = S + d * ld + j;
      row[0] = v.x; row[1] = v.y; row[2] = v.z; row[3] = v.w;
    }
  } else {
    for (int idx = threadIdx.x; idx < D * cols_here; idx += blockDim.x) {
      const int d = idx / cols_here, j = idx - d * cols_here;
      S[d * ld + j] = mine[static_cast<size_t>(d) * Dv + col0 + j];
    }
  }
}
__device__ __forceinline__ void store_state_slice(const float* S, int ld, float* mine, int D, int Dv, int col0, int cols_here) {
  if ((Dv & 3) == 0 && (col0 & 3) == 0 && (cols_here & 3) == 0 && (reinterpret_cast<uintptr_t>(mine) & 15) == 0) {
    const int quads = cols_here >> 2;
    for (int idx = threadIdx.x; idx < D * quads; idx += blockDim.x) {
      const int d = idx / quads, j = (idx - d * quads) << 2;
      const float* row = S + d * ld + j;
      *reinterpret_cast<float4*>(mine + static_cast<size_t>(d) * Dv + col0 + j) = make_float4(row[0], row[1], row[2], row[3]);
    }
  } else {
    for (int idx = threadIdx.x; idx < D * cols_here; idx += blockDim.x) {
      const int d = idx / cols_here, c = idx - d * cols_here;
      mine[static_cast<size_t>(d) * Dv + col0 + c] = S[d * ld + c];
    }
  }
}

__device__ __forceinline__ float log_sigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

__global__ void matrix_memory_scan_kernel(const ScanArgs a) {
  extern __shared__ float scan_shared[];
  let_dependents_start();
  wait_for_previous();
  const int seq = blockIdx.z, head = blockIdx.y, col0 = blockIdx.x * a.cols;
  const int slot = a.state_slot[seq];
  const int start = a.q_start[seq], count = a.q_start[seq + 1] - start;
  const int cols_here = min(a.cols, a.vdim - col0);
  if (slot < 0 || slot >= a.num_slots) {
    // a padding row of the batch: no state is touched; its outputs are made finite (0 over 1) for the kernels after
    for (int idx = threadIdx.x; idx < count * cols_here; idx += blockDim.x) {
      const int t = idx / cols_here, c = idx - t * cols_here;
      a.numerator[(static_cast<size_t>(start + t) * a.heads + head) * a.vdim + col0 + c] = 0.f;
    }
    if (blockIdx.x == 0)
      for (int t = threadIdx.x; t < count; t += blockDim.x) a.denominator[static_cast<size_t>(start + t) * a.heads + head] = 1.f;
    return;
  }
  const bool keeps_z = blockIdx.x == 0;
  const int ld = a.cols + 1;
  const int D = a.dim, Dv = a.vdim, H = a.heads;
  float* S = scan_shared;                           // [D][ld]
  float* qs = S + static_cast<size_t>(D) * ld;      // [TOKENS][D]
  float* ks = qs + SCAN_TOKENS * D;                 // [TOKENS][D]
  float* vs = ks + SCAN_TOKENS * D;                 // [TOKENS][cols]
  float* gates = vs + SCAN_TOKENS * a.cols;         // [TOKENS][2]: input gate, log forget gate
  float* mine = a.state + (static_cast<size_t>(slot) * H + head) * static_cast<size_t>(a.head_stride);
  load_state_slice(S, ld, mine, D, Dv, col0, cols_here);
  if (keeps_z)
    for (int d = threadIdx.x; d < D; d += blockDim.x) S[d * ld + a.cols] = mine[static_cast<size_t>(D) * Dv + d];
  float m = mine[static_cast<size_t>(D) * Dv + D];
  const int j = threadIdx.x;
  const bool value_column = j < cols_here, z_column = keeps_z && j == a.cols;
  const int q_cols = H * D, v_first = 2 * q_cols, gate_first = 2 * q_cols + 2 * H * Dv;
  for (int t0 = 0; t0 < count; t0 += SCAN_TOKENS) {
    const int here = min(SCAN_TOKENS, count - t0);
    __syncthreads();
    for (int idx = threadIdx.x; idx < here * D; idx += blockDim.x) {
      const int t = idx / D, d = idx - t * D;
      const float* row = a.fused + static_cast<size_t>(start + t0 + t) * a.total;
      qs[t * D + d] = __fmul_rn(sum_partials(row + head * D + d, a.stride, a.partials), a.q_scale);
      ks[t * D + d] = sum_partials(row + q_cols + head * D + d, a.stride, a.partials);
    }
    for (int idx = threadIdx.x; idx < here * cols_here; idx += blockDim.x) {
      const int t = idx / cols_here, c = idx - t * cols_here;
      const float* row = a.fused + static_cast<size_t>(start + t0 + t) * a.total;
      vs[t * a.cols + c] = sum_partials(row + v_first + head * Dv + col0 + c, a.stride, a.partials);
    }
    for (int idx = threadIdx.x; idx < here * 2; idx += blockDim.x) {
      const int t = idx >> 1, which = idx & 1;
      const float* row = a.fused + static_cast<size_t>(start + t0 + t) * a.total;
      float z = sum_partials(row + gate_first + which * H + head, a.stride, a.partials);
      if (a.gate_bias != nullptr) z = __fadd_rn(z, a.gate_bias[which * H + head]);
      z = a.cap * tanhf(z / a.cap);
      gates[t * 2 + which] = which == 0 ? z : log_sigmoid(z);
    }
    __syncthreads();
    for (int t = 0; t < here; ++t) {
      const float gate_in = gates[t * 2], gate_forget = gates[t * 2 + 1];
      const float m_new = fmaxf(gate_forget + m, gate_in);
      const float keep = expf(gate_forget + m - m_new), take = expf(gate_in - m_new);
      m = m_new;
      if (value_column || z_column) {
        const float tv = z_column ? take : __fmul_rn(take, vs[t * a.cols + j]);
        const float* q = qs + t * D;
        const float* k = ks + t * D;
        float acc = 0.f;
        for (int d = 0; d < D; ++d) {
          const float s = __fmaf_rn(tv, k[d], __fmul_rn(keep, S[d * ld + j]));
          S[d * ld + j] = s;
          acc = __fmaf_rn(s, q[d], acc);
        }
        const size_t token = static_cast<size_t>(start + t0 + t);
        if (z_column) a.denominator[token * H + head] = fmaxf(fabsf(acc), expf(-m)) + a.floor_;
        else a.numerator[(token * H + head) * Dv + col0 + j] = acc;
      }
    }
  }
  __syncthreads();
  store_state_slice(S, ld, mine, D, Dv, col0, cols_here);
  if (keeps_z) {
    for (int d = threadIdx.x; d < D; d += blockDim.x) mine[static_cast<size_t>(D) * Dv + d] = S[d * ld + a.cols];
    if (threadIdx.x == 0) mine[static_cast<size_t>(D) * Dv + D] = m;
  }
}

// ------------------------------------------------------------------------------------ matrix memory: chunks
// The same recurrence for portions, as products over chunks of CHUNK tokens, every chunk on a CTA of its own.
// With b_t the sum of the log forget gates from the chunk's start through token t, g_s = a_s - b_s,
// N_t = max_{s <= t} g_s and M_t = max(m_0, N_t) (m_0: the running maximum the chunk starts from), the recurrence
// unrolls to m_t = b_t + M_t and
//   S_t^T q_t = exp(m_0 - M_t) S_0^T q_t + exp(N_t - M_t) sum_{s <= t} exp(g_s - N_t) (q_t . k_s) v_s
//   S_L       = exp(m_0 - M_L) S_0 + exp(N_L - M_L) sum_s exp(g_s - N_L) k_s v_s^T      (z likewise, with v = 1)
// where every exponent is <= 0.  Four launches:
//   scores  every chunk by itself, once a head: the decayed scores exp(g_s - N_t) (q_t . k_s), N_t, b_t
//   local   every chunk and slice of value columns: what the scores give (the second sum above and its normaliser,
//           into the output buffers) and the chunk's own addition to the state (the last sum)
//   carry   per sequence, head and column slice, chunk after chunk: the state each chunk starts from (written where
//           the chunk's addition was) and its m_0; the state after the last chunk goes to the request's slot
//   finish  every chunk by itself again: adds the part that comes from the state the chunk started from
// All of it float32 on the CUDA cores: the state and what enters it stay 32-bit.  A chunk is the tokens
// [64 c, 64 c + 64) of its sequence's portion; the grid holds ceil(N / 64) + sequences CTAs a head and slice, and a
// CTA finds its sequence by walking the batch's lengths.
constexpr int CHUNK = 64;
constexpr int CHUNK_COLS = 32;
constexpr int CHUNK_THREADS = 256;

struct ChunkArgs {
  ScanArgs scan;
  float* chunk_state;     // [chunks][H][D Dv + D]: a chunk's addition to S and z, then the state it starts from
  float* chunk_info;      // [chunks][H][4]: N_L, b_L, m_0
  float* token_info;      // [N][H][4]: N_t, b_t, exp(g_t - N_L)
  float* chunk_scores;    // [chunks][H][CHUNK][CHUNK]: the decayed scores
  int num_seqs;
};

// (sequence, first token of the chunk within the batch, tokens in the chunk, index of the sequence's first chunk) of
// chunk number `chunk` of the batch; false when the batch has fewer chunks.
__device__ __forceinline__ bool find_chunk(const int* q_start, int num_seqs, int chunk, int* seq, int* first, int* here, int* base) {
  int before = 0;
  for (int s = 0; s < num_seqs; ++s) {
    const int start = q_start[s], count = q_start[s + 1] - start;
    const int chunks = (count + CHUNK - 1) / CHUNK;
    if (chunk < before + chunks) {
      const int c = chunk - before;
      *seq = s;
      *first = start + c * CHUNK;
      *here = min(CHUNK, count - c * CHUNK);
      *base = before;
      return true;
    }
    before += chunks;
  }
  return false;
}

// rows [first, first + here) of a fused projection's columns [col, col + width) into shared memory (row stride ld),
// each times `scale`, rows past `here` zeroed; 16 bytes at a time where the layout allows
__device__ __forceinline__ void load_rows(float* dst, int ld, const ScanArgs& a, int first, int here, int col, int width, float scale) {
  if (ld > width && ld - width < 4)   // rows padded to a multiple of four: the padding reads as zeros
    for (int idx = threadIdx.x; idx < CHUNK * (ld - width); idx += blockDim.x) dst[(idx / (ld - width)) * ld + width + idx % (ld - width)] = 0.f;
  const bool wide = a.partials == 1 && (width & 3) == 0 && (col & 3) == 0 && (a.total & 3) == 0 &&
                    (reinterpret_cast<uintptr_t>(a.fused) & 15) == 0;
  if (wide) {
    const int quads = width >> 2;
    for (int idx = threadIdx.x; idx < CHUNK * quads; idx += blockDim.x) {
      const int t = idx / quads, j = (idx - t * quads) << 2;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (t < here) v = *reinterpret_cast<const float4*>(a.fused + static_cast<size_t>(first + t) * a.total + col + j);
      float* row = dst + t * ld + j;
      row[0] = v.x * scale; row[1] = v.y * scale; row[2] = v.z * scale; row[3] = v.w * scale;
    }
  } else {
    for (int idx = threadIdx.x; idx < CHUNK * width; idx += blockDim.x) {
      const int t = idx / width, j = idx - t * width;
      float v = 0.f;
      if (t < here) v = sum_partials(a.fused + static_cast<size_t>(first + t) * a.total + col + j, a.stride, a.partials);
      dst[t * ld + j] = v * scale;
    }
  }
}

// The decayed scores of a chunk, once a head: W[t][s] = exp(g_s - N_t) (q_t . k_s) for s <= t, 0 above the diagonal;
// N_t, b_t and exp(g_t - N_L) of every token, N_L and b_L of the chunk.
__global__ void __launch_bounds__(CHUNK_THREADS) matrix_memory_scores_kernel(const ChunkArgs c) {
  extern __shared__ float chunk_shared[];
  const ScanArgs& a = c.scan;
  let_dependents_start();
  wait_for_previous();
  int seq, first, here, base;
  if (!find_chunk(a.q_start, c.num_seqs, blockIdx.x, &seq, &first, &here, &base)) return;
  const int slot = a.state_slot[seq];
  if (slot < 0 || slot >= a.num_slots) return;
  const int head = blockIdx.y, tid = threadIdx.x;
  const int D = a.dim, Dv = a.vdim, H = a.heads;
  const int ldq = D + 1;
  float* Q = chunk_shared;                       // [CHUNK][ldq]
  float* K = Q + CHUNK * ldq;                    // [CHUNK][ldq]
  float* g_of = K + CHUNK * ldq;                 // [CHUNK] g_s (-inf past the chunk's end)
  float* top_of = g_of + CHUNK;                  // [CHUNK] N_t
  float* forget = top_of + CHUNK;                // [CHUNK] log forget gates
  const int q_cols = H * D, gate_first = 2 * q_cols + 2 * H * Dv;
  load_rows(Q, ldq, a, first, here, head * D, D, a.q_scale);
  load_rows(K, ldq, a, first, here, q_cols + head * D, D, 1.f);
  for (int idx = tid; idx < here * 2; idx += blockDim.x) {
    const int t = idx >> 1, which = idx & 1;
    const float* row = a.fused + static_cast<size_t>(first + t) * a.total;
    float x = sum_partials(row + gate_first + which * H + head, a.stride, a.partials);
    if (a.gate_bias != nullptr) x = __fadd_rn(x, a.gate_bias[which * H + head]);
    x = a.cap * tanhf(x / a.cap);
    if (which == 0) g_of[t] = x; else forget[t] = log_sigmoid(x);
  }
  __syncthreads();
  const size_t chunk_index = static_cast<size_t>(blockIdx.x) * H + head;
  if (tid == 0) {   // the chunk's running sums and maxima: a short walk by one thread
    float b = 0.f, top = -INFINITY;
    for (int t = 0; t < here; ++t) {
      b += forget[t];
      const float g = g_of[t] - b;
      g_of[t] = g;
      top = fmaxf(top, g);
      top_of[t] = top;
      forget[t] = b;
    }
    for (int t = here; t < CHUNK; ++t) { g_of[t] = -INFINITY; top_of[t] = top; }
    c.chunk_info[chunk_index * 4] = top;
    c.chunk_info[chunk_index * 4 + 1] = b;
  }
  __syncthreads();
  if (tid < here) {
    float* info = c.token_info + (static_cast<size_t>(first + tid) * H + head) * 4;
    info[0] = top_of[tid];
    info[1] = forget[tid];
    info[2] = expf(g_of[tid] - top_of[CHUNK - 1]);
  }
  // thread (ty, tx) forms rows ty * 4 + i, columns tx + 16 j
  const int ty = tid >> 4, tx = tid & 15;
  float acc[4][4] = {};
  for (int d = 0; d < D; ++d) {
    float q[4], k[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) q[i] = Q[(ty * 4 + i) * ldq + d];
#pragma unroll
    for (int j = 0; j < 4; ++j) k[j] = K[(tx + 16 * j) * ldq + d];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = __fmaf_rn(q[i], k[j], acc[i][j]);
  }
  float* scores = c.chunk_scores + chunk_index * (CHUNK * CHUNK);
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int t = ty * 4 + i, s = tx + 16 * j;
      scores[t * CHUNK + s] = s <= t ? __fmul_rn(expf(g_of[s] - top_of[t]), acc[i][j]) : 0.f;
    }
}

// What a chunk's own tokens give, for one slice of value columns: the decayed scores times v (and their row sums),
// and the chunk's addition to the state, sum_s exp(g_s - N_L) k_s v_s^T.
__global__ void __launch_bounds__(CHUNK_THREADS) matrix_memory_local_kernel(const ChunkArgs c) {
  extern __shared__ float chunk_shared[];
  const ScanArgs& a = c.scan;
  let_dependents_start();
  wait_for_previous();
  int seq, first, here, base;
  if (!find_chunk(a.q_start, c.num_seqs, blockIdx.x, &seq, &first, &here, &base)) return;
  const int head = blockIdx.y, col0 = blockIdx.z * CHUNK_COLS;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int D = a.dim, Dv = a.vdim, H = a.heads;
  const int cols_here = min(CHUNK_COLS, Dv - col0);
  const bool first_slice = blockIdx.z == 0;
  const int slot = a.state_slot[seq];
  if (slot < 0 || slot >= a.num_slots) {   // a padding row: finite outputs, nothing else
    for (int idx = tid; idx < here * cols_here; idx += blockDim.x) {
      const int t = idx / cols_here, col = idx - t * cols_here;
      a.numerator[(static_cast<size_t>(first + t) * H + head) * Dv + col0 + col] = 0.f;
    }
    if (first_slice)
      for (int t = tid; t < here; t += blockDim.x) a.denominator[static_cast<size_t>(first + t) * H + head] = 1.f;
    return;
  }
  // K and the scores are read here a row at a time by all lanes alike (broadcasts), so their rows keep 16-byte
  // alignment and are read four elements a load
  const int ldq = (D + 3) & ~3, ldw = CHUNK;
  float* K = chunk_shared;                       // [CHUNK][ldq]
  float* V = K + CHUNK * ldq;                    // [CHUNK][CHUNK_COLS]
  float* W = V + CHUNK * CHUNK_COLS;             // [CHUNK][ldw]
  float* take = W + CHUNK * ldw;                 // [CHUNK] exp(g_s - N_L), 0 past the chunk's end
  const int q_cols = H * D, v_first = 2 * q_cols;
  const size_t chunk_index = static_cast<size_t>(blockIdx.x) * H + head;
  load_rows(K, ldq, a, first, here, q_cols + head * D, D, 1.f);
  if (cols_here == CHUNK_COLS) load_rows(V, CHUNK_COLS, a, first, here, v_first + head * Dv + col0, CHUNK_COLS, 1.f);
  else
    for (int idx = tid; idx < CHUNK * CHUNK_COLS; idx += blockDim.x) {
      const int t = idx / CHUNK_COLS, col = idx - t * CHUNK_COLS;
      V[idx] = (t < here && col < cols_here)
                   ? sum_partials(a.fused + static_cast<size_t>(first + t) * a.total + v_first + head * Dv + col0 + col, a.stride, a.partials)
                   : 0.f;
    }
  const float* scores = c.chunk_scores + chunk_index * (CHUNK * CHUNK);
  for (int idx = tid; idx < CHUNK * CHUNK / 4; idx += blockDim.x) {
    const int t = idx / (CHUNK / 4), s = (idx - t * (CHUNK / 4)) * 4;
    const float4 w = *reinterpret_cast<const float4*>(scores + t * CHUNK + s);
    *reinterpret_cast<float4*>(W + t * ldw + s) = w;
  }
  if (tid < CHUNK) take[tid] = tid < here ? c.token_info[(static_cast<size_t>(first + tid) * H + head) * 4 + 2] : 0.f;
  __syncthreads();
  {   // warp w rows w * 8 .. w * 8 + 7, lane its column
    float acc[8] = {};
    const int t_first = warp * 8;
    for (int s = 0; s < min(here, t_first + 8); s += 4) {   // the scores past a row's own token and past the chunk are 0
      float vv[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) vv[k] = V[(s + k) * CHUNK_COLS + lane];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float4 w = *reinterpret_cast<const float4*>(W + (t_first + i) * ldw + s);
        acc[i] = __fmaf_rn(w.x, vv[0], acc[i]);
        acc[i] = __fmaf_rn(w.y, vv[1], acc[i]);
        acc[i] = __fmaf_rn(w.z, vv[2], acc[i]);
        acc[i] = __fmaf_rn(w.w, vv[3], acc[i]);
      }
    }
    if (lane < cols_here) {
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (t_first + i < here) a.numerator[(static_cast<size_t>(first + t_first + i) * H + head) * Dv + col0 + lane] = acc[i];
    }
    if (first_slice && tid < here) {
      float rest = 0.f;
      for (int s = 0; s <= tid; ++s) rest = __fadd_rn(rest, W[tid * ldw + s]);
      a.denominator[static_cast<size_t>(first + tid) * H + head] = rest;
    }
  }
  __syncthreads();
  for (int idx = tid; idx < CHUNK * CHUNK_COLS; idx += blockDim.x) V[idx] = __fmul_rn(V[idx], take[idx / CHUNK_COLS]);
  __syncthreads();
  float* addition = c.chunk_state + chunk_index * (static_cast<size_t>(D) * Dv + D);
  for (int d0 = warp * 8; d0 < D; d0 += 8 * (CHUNK_THREADS / 32)) {   // warp w rows d0 .. d0 + 7, lane its column
    float acc[8] = {};
    const int rows = min(8, D - d0);
    for (int s = 0; s < here; ++s) {
      const float vv = V[s * CHUNK_COLS + lane];
      // K's rows are padded to a multiple of four (zeros), so both loads stay inside the row
      const float4 lo = *reinterpret_cast<const float4*>(K + s * ldq + d0);
      const float4 hi = rows > 4 ? *reinterpret_cast<const float4*>(K + s * ldq + d0 + 4) : make_float4(0.f, 0.f, 0.f, 0.f);
      acc[0] = __fmaf_rn(lo.x, vv, acc[0]); acc[1] = __fmaf_rn(lo.y, vv, acc[1]);
      acc[2] = __fmaf_rn(lo.z, vv, acc[2]); acc[3] = __fmaf_rn(lo.w, vv, acc[3]);
      acc[4] = __fmaf_rn(hi.x, vv, acc[4]); acc[5] = __fmaf_rn(hi.y, vv, acc[5]);
      acc[6] = __fmaf_rn(hi.z, vv, acc[6]); acc[7] = __fmaf_rn(hi.w, vv, acc[7]);
    }
    if (lane < cols_here) {
#pragma unroll
      for (int r = 0; r < 8; ++r)
        if (r < rows) addition[static_cast<size_t>(d0 + r) * Dv + col0 + lane] = acc[r];
    }
  }
  if (first_slice)
    for (int d = tid; d < D; d += blockDim.x) {
      float acc = 0.f;
      for (int s = 0; s < here; ++s) acc = __fmaf_rn(take[s], K[s * ldq + d], acc);
      addition[static_cast<size_t>(D) * Dv + d] = acc;
    }
}

constexpr int CARRY_ROWS = 64;         // rows of a state slice one CTA of the carry kernel holds
constexpr int CARRY_PER_THREAD = CARRY_ROWS * CHUNK_COLS / CHUNK_THREADS;

// Elementwise and in order: a CTA holds CARRY_ROWS rows of one column slice of one head's state in registers and
// walks the sequence's chunks; the next chunk's addition is on its way while this one's is used.
__global__ void __launch_bounds__(CHUNK_THREADS) matrix_memory_carry_kernel(const ChunkArgs c, int row_groups) {
  const ScanArgs& a = c.scan;
  let_dependents_start();
  wait_for_previous();
  const int seq = blockIdx.z, head = blockIdx.y;
  const int slice = blockIdx.x / row_groups, row0 = (blockIdx.x - slice * row_groups) * CARRY_ROWS, col0 = slice * CHUNK_COLS;
  const int slot = a.state_slot[seq];
  if (slot < 0 || slot >= a.num_slots) return;
  const int D = a.dim, Dv = a.vdim, H = a.heads, tid = threadIdx.x;
  const int cols_here = min(CHUNK_COLS, Dv - col0);
  const bool holds_z = slice == 0, writes_info = blockIdx.x == 0;
  int base = 0;   // the sequence's first chunk
  for (int s = 0; s < seq; ++s) base += (a.q_start[s + 1] - a.q_start[s] + CHUNK - 1) / CHUNK;
  const int chunks = (a.q_start[seq + 1] - a.q_start[seq] + CHUNK - 1) / CHUNK;
  float* mine = a.state + (static_cast<size_t>(slot) * H + head) * static_cast<size_t>(a.head_stride);
  const size_t per_chunk = static_cast<size_t>(D) * Dv + D;
  // element i of a thread: row row0 + (tid + i * 256) / 32, column col0 + tid % 32
  const int col = tid & (CHUNK_COLS - 1);
  size_t offset[CARRY_PER_THREAD];
  bool live[CARRY_PER_THREAD];
  float held[CARRY_PER_THREAD], next[CARRY_PER_THREAD], held_z = 0.f, next_z = 0.f;
#pragma unroll
  for (int i = 0; i < CARRY_PER_THREAD; ++i) {
    const int row = row0 + (tid + i * CHUNK_THREADS) / CHUNK_COLS;
    live[i] = row < D && col < cols_here;
    offset[i] = static_cast<size_t>(row) * Dv + col0 + col;
    held[i] = live[i] ? mine[offset[i]] : 0.f;
  }
  const bool z_live = holds_z && tid < CARRY_ROWS && row0 + tid < D;
  const size_t z_offset = static_cast<size_t>(D) * Dv + row0 + tid;
  if (z_live) held_z = mine[z_offset];
  float m0 = mine[static_cast<size_t>(D) * Dv + D];
  float* addition = c.chunk_state + (static_cast<size_t>(base) * H + head) * per_chunk;
  const float* info = c.chunk_info + (static_cast<size_t>(base) * H + head) * 4;
  float top = 0.f, b = 0.f;
  if (chunks > 0) {
    top = info[0];
    b = info[1];
#pragma unroll
    for (int i = 0; i < CARRY_PER_THREAD; ++i) next[i] = live[i] ? addition[offset[i]] : 0.f;
    if (z_live) next_z = addition[z_offset];
  }
  for (int k = 0; k < chunks; ++k) {
    float added[CARRY_PER_THREAD], added_z = next_z;
#pragma unroll
    for (int i = 0; i < CARRY_PER_THREAD; ++i) added[i] = next[i];
    const float top_now = top, b_now = b;
    float* here = addition;
    if (k + 1 < chunks) {   // the next chunk's figures, asked for before this chunk's are used
      addition += static_cast<size_t>(H) * per_chunk;
      info += static_cast<size_t>(H) * 4;
      top = info[0];
      b = info[1];
#pragma unroll
      for (int i = 0; i < CARRY_PER_THREAD; ++i) next[i] = live[i] ? addition[offset[i]] : 0.f;
      if (z_live) next_z = addition[z_offset];
    }
    const float top_all = fmaxf(m0, top_now);
    const float keep = expf(m0 - top_all), take = expf(top_now - top_all);
#pragma unroll
    for (int i = 0; i < CARRY_PER_THREAD; ++i)
      if (live[i]) {
        here[offset[i]] = held[i];   // the state this chunk starts from
        held[i] = __fmaf_rn(keep, held[i], __fmul_rn(take, added[i]));
      }
    if (z_live) {
      here[z_offset] = held_z;
      held_z = __fmaf_rn(keep, held_z, __fmul_rn(take, added_z));
    }
    if (writes_info && tid == 0) c.chunk_info[(static_cast<size_t>(base + k) * H + head) * 4 + 2] = m0;
    m0 = b_now + top_all;
  }
#pragma unroll
  for (int i = 0; i < CARRY_PER_THREAD; ++i)
    if (live[i]) mine[offset[i]] = held[i];
  if (z_live) mine[z_offset] = held_z;
  if (writes_info && tid == 0) mine[static_cast<size_t>(D) * Dv + D] = m0;
}

__global__ void __launch_bounds__(CHUNK_THREADS) matrix_memory_finish_kernel(const ChunkArgs c) {
  extern __shared__ float chunk_shared[];
  const ScanArgs& a = c.scan;
  let_dependents_start();
  wait_for_previous();
  int seq, first, here, base;
  if (!find_chunk(a.q_start, c.num_seqs, blockIdx.x, &seq, &first, &here, &base)) return;
  const int slot = a.state_slot[seq];
  if (slot < 0 || slot >= a.num_slots) return;
  const int head = blockIdx.y, col0 = blockIdx.z * CHUNK_COLS;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int D = a.dim, Dv = a.vdim, H = a.heads;
  const int cols_here = min(CHUNK_COLS, Dv - col0);
  const bool first_slice = blockIdx.z == 0;
  const int ldq = (D + 3) & ~3, lds = CHUNK_COLS + 1;   // Q's rows are read by all lanes alike: 16-byte aligned, four a load
  float* Q = chunk_shared;                       // [CHUNK][ldq]
  float* S = Q + CHUNK * ldq;                    // [D][lds]: the state the chunk starts from
  float* z = S + static_cast<size_t>(D) * lds;   // [D]
  const size_t chunk_index = static_cast<size_t>(blockIdx.x) * H + head;
  const float* before = c.chunk_state + chunk_index * (static_cast<size_t>(D) * Dv + D);
  const float m0 = c.chunk_info[chunk_index * 4 + 2];
  load_rows(Q, ldq, a, first, here, head * D, D, a.q_scale);
  if (cols_here < CHUNK_COLS) {
    for (int idx = tid; idx < D * lds; idx += blockDim.x) S[idx] = 0.f;
    __syncthreads();
  }
  load_state_slice(S, lds, before, D, Dv, col0, cols_here);
  if (first_slice)
    for (int d = tid; d < D; d += blockDim.x) z[d] = before[static_cast<size_t>(D) * Dv + d];
  __syncthreads();
  float acc[8] = {};
  const int t_first = warp * 8;
  for (int d = 0; d < D; d += 4) {   // Q's columns past D are zero, S's rows past D are never reached by a nonzero
    float sv[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) sv[k] = d + k < D ? S[(d + k) * lds + lane] : 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float4 q = *reinterpret_cast<const float4*>(Q + (t_first + i) * ldq + d);
      acc[i] = __fmaf_rn(q.x, sv[0], acc[i]);
      acc[i] = __fmaf_rn(q.y, sv[1], acc[i]);
      acc[i] = __fmaf_rn(q.z, sv[2], acc[i]);
      acc[i] = __fmaf_rn(q.w, sv[3], acc[i]);
    }
  }
  if (lane < cols_here) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int t = t_first + i;
      if (t < here) {
        const size_t token = static_cast<size_t>(first + t) * H + head;
        const float top = c.token_info[token * 4], top_all = fmaxf(m0, top);
        float* out = a.numerator + token * Dv + col0 + lane;
        *out = __fmaf_rn(expf(m0 - top_all), acc[i], __fmul_rn(expf(top - top_all), *out));
      }
    }
  }
  if (first_slice && tid < here) {
    const size_t token = static_cast<size_t>(first + tid) * H + head;
    float dot = 0.f;
    for (int d = 0; d < D; ++d) dot = __fmaf_rn(Q[tid * ldq + d], z[d], dot);
    const float top = c.token_info[token * 4], b = c.token_info[token * 4 + 1], top_all = fmaxf(m0, top);
    const float nq = __fmaf_rn(expf(m0 - top_all), dot, __fmul_rn(expf(top - top_all), a.denominator[token]));
    a.denominator[token] = fmaxf(fabsf(nq), expf(-(b + top_all))) + a.floor_;
  }
}

// Shared memory of the chunk kernels for heads of `dim`; 0 when they do not fit (the walk serves those).
static size_t chunk_smem_bytes(int dim, size_t* scores_bytes, size_t* finish_bytes) {
  *scores_bytes = (2ull * CHUNK * (dim + 1) + 3 * CHUNK) * sizeof(float);
  const size_t padded = (static_cast<size_t>(dim) + 3) & ~static_cast<size_t>(3);
  const size_t local = (CHUNK * padded + CHUNK * CHUNK_COLS + static_cast<size_t>(CHUNK) * CHUNK + CHUNK) * sizeof(float);
  *finish_bytes = (CHUNK * padded + (padded + 4) * (CHUNK_COLS + 1) + padded) * sizeof(float);
  const size_t limit = static_cast<size_t>(shrike_device().max_smem);
  return (local <= limit && *finish_bytes <= limit && *scores_bytes <= limit) ? local : 0;
}

// -------------------------------------------------------------------------------------- matrix memory: out
struct MemoryOutArgs {
  const float* numerator;    // [N][H][Dv]
  const float* denominator;  // [N][H]
  const float* fused;        // the projection the scan read; its gate columns start at `gate_first`
  long long stride;
  int partials, total, gate_first;
  const float* weight;       // [H Dv]
  float eps;
  void* out;                 // [N][H Dv]
  int n, heads, vdim;
};

template <typename T>
__global__ void __launch_bounds__(PREP_WARPS * 32) matrix_memory_out_kernel(const MemoryOutArgs a) {
  let_dependents_start();
  wait_for_previous();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long work = static_cast<long long>(blockIdx.x) * PREP_WARPS + warp;
  if (work >= static_cast<long long>(a.n) * a.heads) return;
  const int token = static_cast<int>(work / a.heads), head = static_cast<int>(work - static_cast<long long>(token) * a.heads);
  const float* num = a.numerator + static_cast<size_t>(work) * a.vdim;
  const float inv = 1.0f / a.denominator[work];
  float squares = 0.f;
  for (int c = lane; c < a.vdim; c += 32) {
    const float o = __fmul_rn(num[c], inv);
    squares = __fmaf_rn(o, o, squares);
  }
  const float r = rsqrtf(warp_sum(squares) / static_cast<float>(a.vdim) + a.eps);
  const float* gate_row = a.fused + static_cast<size_t>(token) * a.total + a.gate_first + head * a.vdim;
  T* out = static_cast<T*>(a.out) + (static_cast<size_t>(token) * a.heads + head) * a.vdim;
  for (int c = lane; c < a.vdim; c += 32) {
    const float gate = 1.0f / (1.0f + expf(-sum_partials(gate_row + c, a.stride, a.partials)));
    out[c] = from_float<T>(__fmul_rn(num[c], inv) * r * a.weight[head * a.vdim + c] * gate);
  }
}

// ----------------------------------------------------------------------------------------------- route_top
// One block a token.  The logits: the block's warps share a row's columns (warp w the w-th run of 128 columns, and
// so on), experts eight at a time with the eight weight rows' loads in flight together; the warps' sums meet in shared
// memory in a fixed order.  Then, by the first warp: softmax, `top` rounds of a warp-wide argmax, the sum of the
// chosen, and the shared expert's gate (its vector is one more row of the product).
constexpr int ROUTE_WARPS = 8;
constexpr int ROUTE_GROUP = 8;

template <typename T>
__global__ void __launch_bounds__(ROUTE_WARPS * 32)
route_top_kernel(const T* __restrict__ x, const float* __restrict__ router, const float* __restrict__ shared_gate,
                 float* __restrict__ weights, int n, int width, int experts, int top, int columns, float renorm_eps,
                 int sigmoid_scores, int renormalise) {
  extern __shared__ float route_shared[];   // [ROUTE_WARPS][rows] sums of the warps, then [rows] scores in the first row
  let_dependents_start();
  wait_for_previous();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int token = blockIdx.x;
  const T* row = x + static_cast<size_t>(token) * width;
  float* out = weights + static_cast<size_t>(token) * columns;
  // rows of the product: the experts, then (when there is one) the shared expert's gate vector
  const int rows = experts + (columns > experts && shared_gate != nullptr ? 1 : 0);
  const bool wide = (width & 3) == 0 && (reinterpret_cast<uintptr_t>(router) & 15) == 0 &&
                    (shared_gate == nullptr || (reinterpret_cast<uintptr_t>(shared_gate) & 15) == 0) &&
                    (reinterpret_cast<uintptr_t>(x) & 15) == 0;
  float* partial = route_shared + static_cast<size_t>(warp) * rows;
  for (int e0 = 0; e0 < rows; e0 += ROUTE_GROUP) {
    float dot[ROUTE_GROUP] = {};
    const float* from[ROUTE_GROUP];
#pragma unroll
    for (int g = 0; g < ROUTE_GROUP; ++g) {
      const int e = min(e0 + g, rows - 1);   // rows past the end repeat the last one; their sums are dropped
      from[g] = e < experts ? router + static_cast<size_t>(e) * width : shared_gate;
    }
    if (wide) {
#pragma unroll 2
      for (int c = (warp * 32 + lane) * 4; c < width; c += ROUTE_WARPS * 128) {
        float xv[4], w[ROUTE_GROUP][4];
        load4<T>(row + c, xv);
#pragma unroll
        for (int g = 0; g < ROUTE_GROUP; ++g) load4<float>(from[g] + c, w[g]);
#pragma unroll
        for (int g = 0; g < ROUTE_GROUP; ++g)
#pragma unroll
          for (int k = 0; k < 4; ++k) dot[g] = __fmaf_rn(xv[k], w[g][k], dot[g]);
      }
    } else {
      for (int c = warp * 32 + lane; c < width; c += ROUTE_WARPS * 32) {
        const float xv = to_float(row[c]);
#pragma unroll
        for (int g = 0; g < ROUTE_GROUP; ++g) dot[g] = __fmaf_rn(xv, from[g][c], dot[g]);
      }
    }
#pragma unroll
    for (int g = 0; g < ROUTE_GROUP; ++g) {
      const float sum = warp_sum(dot[g]);
      if (lane == 0 && e0 + g < rows) partial[e0 + g] = sum;
    }
  }
  __syncthreads();
  if (warp != 0) return;
  float* score = route_shared;
  float best = -INFINITY;
  for (int e = lane; e < rows; e += 32) {
    float sum = score[e];
    for (int w = 1; w < ROUTE_WARPS; ++w) sum = __fadd_rn(sum, route_shared[static_cast<size_t>(w) * rows + e]);
    score[e] = sum;
    if (e < experts) best = fmaxf(best, sum);
  }
  best = warp_max(best);
  __syncwarp();
  const float shared_dot = rows > experts ? score[experts] : 0.f;
  float total = 0.f;
  for (int e = lane; e < experts; e += 32) {
    // an expert's score: its share of the softmax over all experts, or the sigmoid of its own logit.  The sigmoid is
    // taken when an expert is chosen: the choice itself goes by the logits, which order the experts as their sigmoids
    // do and do not run together where the sigmoid rounds to 1 or to 0
    const float p = sigmoid_scores ? score[e] : expf(score[e] - best);
    score[e] = p;
    total += p;
  }
  total = sigmoid_scores ? 1.f : warp_sum(total);
  __syncwarp();
  for (int e = lane; e < experts; e += 32) {
    score[e] = score[e] / total;
    out[e] = 0.f;
  }
  __syncwarp();
  float chosen_sum = 0.f;
  // `top` rounds of a warp-wide argmax; the lowest index wins a tie.  A pick is marked by a value below every score.
  const float below = sigmoid_scores ? -INFINITY : -1.f;
  for (int round = 0; round < top; ++round) {
    float mine = below;
    int where = experts;
    for (int e = lane; e < experts; e += 32)
      if (score[e] > mine) { mine = score[e]; where = e; }
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
      const float other = __shfl_xor_sync(0xffffffffu, mine, offset);
      const int other_where = __shfl_xor_sync(0xffffffffu, where, offset);
      if (other > mine || (other == mine && other_where < where)) { mine = other; where = other_where; }
    }
    if (sigmoid_scores) mine = 1.0f / (1.0f + expf(-mine));
    chosen_sum += mine;
    if (lane == 0 && where < experts) {
      out[where] = mine;
      score[where] = sigmoid_scores ? -INFINITY : -2.f;
    }
    __syncwarp();
  }
  if (renormalise) {
    const float inv = 1.0f / (chosen_sum + renorm_eps);
    for (int e = lane; e < experts; e += 32) out[e] = out[e] * inv;
  }
  if (columns > experts && lane == 0) out[experts] = shared_gate != nullptr ? 1.0f / (1.0f + expf(-shared_dot)) : 1.f;
}

// ------------------------------------------------------------------------------------------ act_mul_blocks
// gate_up [N][2 I]: all gate columns, then all up columns; I = experts * each + rest.  Column c belongs to
// expert c / each, the last `rest` columns to the shared expert (weight column `experts`).
template <typename T, int VEC>
__global__ void __launch_bounds__(256)
act_mul_blocks_kernel(const T* __restrict__ gate_up, const float* __restrict__ weights, T* __restrict__ out, int n, int inter,
                      int experts, int each, int columns, int act, float limit, int weight_input) {
  let_dependents_start();
  wait_for_previous();
  // VEC consecutive columns a thread (one 16-byte access each way when VEC > 1; the launcher sees to it that a
  // group never straddles two experts)
  struct alignas(sizeof(T) * VEC) Pack { T v[VEC]; };
  const int groups = inter / VEC;
  for (int row = blockIdx.y; row < n; row += gridDim.y) {
    const T* in = gate_up + static_cast<size_t>(row) * 2 * inter;
    const float* w = weights + static_cast<size_t>(row) * columns;
    T* o = out + static_cast<size_t>(row) * inter;
    for (int group = blockIdx.x * blockDim.x + threadIdx.x; group < groups; group += gridDim.x * blockDim.x) {
      const int c = group * VEC;
      const int block = c < experts * each ? c / each : experts;
      const float share = w[block];
      Pack r;
      if (share == 0.f) {
        // an expert the token did not choose contributes exactly nothing, whatever its gate and up columns hold
#pragma unroll
        for (int j = 0; j < VEC; ++j) r.v[j] = from_float<T>(0.f);
      } else {
        const Pack g = *reinterpret_cast<const Pack*>(in + c), u = *reinterpret_cast<const Pack*>(in + inter + c);
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
          // the weight on the expert's INPUT reaches gate and up alike (both are linear in it): act(w g) (w u)
          const float gate = to_float(g.v[j]), up = to_float(u.v[j]);
          r.v[j] = from_float<T>(weight_input ? act_times<T>(act, __fmul_rn(share, gate), __fmul_rn(share, up), limit)
                                              : __fmul_rn(act_times<T>(act, gate, up, limit), share));
        }
      }
      *reinterpret_cast<Pack*>(o + c) = r;
    }
  }
}

}  // namespace parallel

// =========================================================================================== launchers
using namespace parallel;

// terms: `num_terms` (at most 4) pending sums, term t = data[t] ([partials[t]][N][W] float32, `strides[t]` elements
// between partials) times scales[t].  norms: 0..2, norm k = tanh(alpha[k] x) * weight[k] + bias[k] into out[k]
// ([N or R][W] of out_dtype).  rows null: resid is rewritten with the sum; else only out[k][r] for row rows[r].
SHRIKE_API int shrike_tanh_norm(float* resid, const float* const* data, const int* partials, const long long* strides,
                                const float* scales, int num_terms, const float* row_add, const int* rows, int norms,
                                const float* alpha, const float* const* weight, const float* const* bias, void* const* out,
                                int out_dtype, int n, int width, cudaStream_t stream) {
  if (n <= 0) return SHRIKE_OK;
  if (width <= 0 || num_terms < 0 || num_terms > MAX_TERMS || norms < 0 || norms > 2) return SHRIKE_BAD_ARGUMENT;
  if (norms > 0 && out_dtype != SHRIKE_F32 && out_dtype != SHRIKE_BF16) return SHRIKE_BAD_ARGUMENT;
  TanhNormArgs a = {};
  a.resid = resid;
  a.num_terms = num_terms;
  for (int t = 0; t < num_terms; ++t) {
    if (partials[t] < 1) return SHRIKE_BAD_ARGUMENT;
    a.terms[t] = SumTerm{data[t], strides[t], partials[t], scales[t]};
  }
  a.row_add = row_add;
  a.rows = rows;
  a.norms = norms;
  for (int k = 0; k < norms; ++k) {
    a.alpha[k] = alpha[k];
    a.weight[k] = weight[k];
    a.bias[k] = bias[k];
    a.out[k] = out[k];
  }
  a.n = n;
  a.width = width;
  bool vec = width % 4 == 0 && (reinterpret_cast<uintptr_t>(resid) & 15) == 0 && (reinterpret_cast<uintptr_t>(row_add) & 15) == 0;
  for (int t = 0; t < num_terms; ++t) vec = vec && (reinterpret_cast<uintptr_t>(data[t]) & 15) == 0 && strides[t] % 4 == 0;
  for (int k = 0; k < norms; ++k)
    vec = vec && ((reinterpret_cast<uintptr_t>(weight[k]) | reinterpret_cast<uintptr_t>(bias[k]) | reinterpret_cast<uintptr_t>(out[k])) & 15) == 0;
  const int groups = vec ? width / 4 : width;
  const dim3 grid(max(1, min(32, (groups + 255) / 256)), max(1, min(n, 65535)));
  const bool bf16 = norms > 0 && out_dtype == SHRIKE_BF16;
  if (vec && bf16) launch_dependent(tanh_norm_kernel<__nv_bfloat16, 4>, grid, 256, 0, stream, a);
  else if (vec) launch_dependent(tanh_norm_kernel<float, 4>, grid, 256, 0, stream, a);
  else if (bf16) launch_dependent(tanh_norm_kernel<__nv_bfloat16, 1>, grid, 256, 0, stream, a);
  else launch_dependent(tanh_norm_kernel<float, 1>, grid, 256, 0, stream, a);
  return shrike_launch_status();
}

// `whole_norm`: q and k over the root mean square of their whole projections, the weights one number a column.
// `value_norm`: every value head over its own root mean square.  `kv_heads` 0: the projection holds queries alone
// (a layer that reads another layer's keys and values).
SHRIKE_API int shrike_head_prep_norms(const float* fused, int partials, long long stride, int total, const float* bias,
                                      const int* positions, const float* inv_freq, int rot, const float* q_weight,
                                      const float* k_weight, float eps, void* q_out, void* keys, void* values, const int* slots,
                                      float* gate_out, int dtype, int n, int heads, int kv_heads, int dim, int vdim, int padded,
                                      int num_slots, int whole_norm, int value_norm, cudaStream_t stream) {
  if (n <= 0) return SHRIKE_OK;
  if (heads < 1 || kv_heads < 0 || dim < 1 || vdim < 1 || padded < dim || padded < vdim || partials < 1 || rot < 0 ||
      rot % 2 || rot > dim || padded > 8192)
    return SHRIKE_BAD_ARGUMENT;
  if (total < heads * dim + kv_heads * (dim + vdim) + (gate_out != nullptr ? heads : 0)) return SHRIKE_BAD_ARGUMENT;
  HeadPrepArgs a = {fused, stride, partials, total, bias, positions, inv_freq, rot, q_weight, k_weight, eps, q_out, keys,
                    values, slots, gate_out, n, heads, kv_heads, dim, vdim, padded, num_slots, whole_norm, value_norm};
  const int units = heads + 2 * kv_heads + (gate_out != nullptr ? 1 : 0);
  // few tokens: a warp a unit, so that a step's heads are all under way at once; many: a block a token
  const int per_token = n >= 1024 ? 1 : (units + PREP_WARPS - 1) / PREP_WARPS;
  if (n > 2147483647 / 2 || per_token > 65535) return SHRIKE_BAD_ARGUMENT;
  const dim3 blocks(static_cast<unsigned>(n), static_cast<unsigned>(per_token));
  const size_t smem = (static_cast<size_t>(PREP_WARPS) * padded + (inv_freq != nullptr ? rot : 0)) * sizeof(float);
  if (dtype == SHRIKE_F32) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(head_prep_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    launch_dependent(head_prep_kernel<float>, blocks, PREP_WARPS * 32, smem, stream, a);
  } else if (dtype == SHRIKE_BF16) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(head_prep_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    launch_dependent(head_prep_kernel<__nv_bfloat16>, blocks, PREP_WARPS * 32, smem, stream, a);
  } else return SHRIKE_BAD_ARGUMENT;
  return shrike_launch_status();
}

SHRIKE_API int shrike_head_prep(const float* fused, int partials, long long stride, int total, const float* bias,
                                const int* positions, const float* inv_freq, int rot, const float* q_weight,
                                const float* k_weight, float eps, void* q_out, void* keys, void* values, const int* slots,
                                float* gate_out, int dtype, int n, int heads, int kv_heads, int dim, int vdim, int padded,
                                int num_slots, cudaStream_t stream) {
  if (kv_heads < 1) return SHRIKE_BAD_ARGUMENT;
  return shrike_head_prep_norms(fused, partials, stride, total, bias, positions, inv_freq, rot, q_weight, k_weight, eps, q_out,
                                keys, values, slots, gate_out, dtype, n, heads, kv_heads, dim, vdim, padded, num_slots, 0, 0, stream);
}

// Value columns a CTA of the scan takes: as many (at most 64) as let the state slice, the staged tokens and a
// second CTA fit an SM's shared memory.
static int scan_columns(int dim, int vdim, size_t* smem_out) {
  const ShrikeDevice& device = shrike_device();
  int cols = vdim < 64 ? vdim : 64;
  for (;;) {
    const size_t floats = static_cast<size_t>(dim) * (cols + 1) + 2ull * SCAN_TOKENS * dim + static_cast<size_t>(SCAN_TOKENS) * cols +
                          2 * SCAN_TOKENS;
    const size_t bytes = floats * sizeof(float);
    if (bytes <= static_cast<size_t>(device.max_smem) / 2 || cols <= 8) {
      *smem_out = bytes;
      return bytes <= static_cast<size_t>(device.max_smem) ? cols : 0;
    }
    cols = (cols + 1) / 2;
  }
}

// `longest`: the most new tokens any sequence of the batch brings.  From CHUNK_FROM on the batch runs on the chunk
// kernels (products over 64 tokens at a time, every chunk on its own CTA), below it on the walk (token by token:
// decoding and short portions).  The chunk kernels need scratch: `chunk_state` (ceil(n / 64) + num_seqs) * heads *
// (dim * vdim + dim) floats, `chunk_info` four floats a chunk and head, `token_info` two a token and head; with any of
// them null the walk runs.  `chunk_scores`: 4096 floats a chunk and head; `token_info`: four a token and head.
constexpr int CHUNK_FROM = 16;

SHRIKE_API long long shrike_matrix_memory_chunks(int n, int num_seqs) { return (static_cast<long long>(n) + CHUNK - 1) / CHUNK + num_seqs; }

SHRIKE_API int shrike_matrix_memory_scan(const float* fused, int partials, long long stride, int total, const float* gate_bias,
                                         float* state, const int* q_start, const int* state_slot, float* numerator,
                                         float* denominator, int num_seqs, int heads, int dim, int vdim, int num_slots,
                                         float cap, float q_scale, float floor_, int longest, int head_stride, int n,
                                         float* chunk_state, float* chunk_info, float* token_info, float* chunk_scores,
                                         cudaStream_t stream) {
  if (num_seqs <= 0) return SHRIKE_OK;
  if (static_cast<long long>(head_stride) < static_cast<long long>(dim) * vdim + dim + 1) return SHRIKE_BAD_ARGUMENT;
  if (heads < 1 || dim < 1 || vdim < 1 || partials < 1 || !(cap > 0.f) || num_seqs > 65535 || heads > 65535) return SHRIKE_BAD_ARGUMENT;
  if (total < 2 * heads * dim + 2 * heads * vdim + 2 * heads) return SHRIKE_BAD_ARGUMENT;
  size_t finish_bytes = 0, scores_bytes = 0;
  const bool scratch = chunk_state != nullptr && chunk_info != nullptr && token_info != nullptr && chunk_scores != nullptr;
  const size_t local_bytes = longest >= CHUNK_FROM && scratch ? chunk_smem_bytes(dim, &scores_bytes, &finish_bytes) : 0;
  const int slices = (vdim + CHUNK_COLS - 1) / CHUNK_COLS;
  if (local_bytes > 0 && slices <= 65535) {
    static bool chunk_configured = false;
    if (!chunk_configured) {
      const int most = shrike_device().max_smem;
      cudaError_t err = cudaFuncSetAttribute(matrix_memory_local_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
      if (err == cudaSuccess) err = cudaFuncSetAttribute(matrix_memory_scores_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
      if (err == cudaSuccess) err = cudaFuncSetAttribute(matrix_memory_finish_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
      if (err != cudaSuccess) return static_cast<int>(err);
      chunk_configured = true;
    }
    ChunkArgs c = {};
    c.scan = ScanArgs{fused, stride, partials, total, gate_bias, state, q_start, state_slot, numerator, denominator,
                      heads, dim, vdim, CHUNK_COLS, num_slots, cap, q_scale, floor_, head_stride};
    c.chunk_state = chunk_state;
    c.chunk_info = chunk_info;
    c.token_info = token_info;
    c.chunk_scores = chunk_scores;
    c.num_seqs = num_seqs;
    const unsigned chunks = static_cast<unsigned>(shrike_matrix_memory_chunks(n, num_seqs));
    launch_dependent(matrix_memory_scores_kernel, dim3(chunks, heads, 1), CHUNK_THREADS, scores_bytes, stream, c);
    launch_dependent(matrix_memory_local_kernel, dim3(chunks, heads, slices), CHUNK_THREADS, local_bytes, stream, c);
    const int row_groups = (dim + CARRY_ROWS - 1) / CARRY_ROWS;
    launch_dependent(matrix_memory_carry_kernel, dim3(slices * row_groups, heads, num_seqs), CHUNK_THREADS, 0, stream, c, row_groups);
    launch_dependent(matrix_memory_finish_kernel, dim3(chunks, heads, slices), CHUNK_THREADS, finish_bytes, stream, c);
    return shrike_launch_status();
  }
  size_t smem = 0;
  const int cols = scan_columns(dim, vdim, &smem);
  if (cols == 0) return SHRIKE_BAD_ARGUMENT;
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    const cudaError_t err = cudaFuncSetAttribute(matrix_memory_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 shrike_device().max_smem);
    if (err != cudaSuccess) return static_cast<int>(err);
    configured = shrike_device().max_smem;
  }
  ScanArgs a = {fused, stride, partials, total, gate_bias, state, q_start, state_slot, numerator, denominator,
                heads, dim, vdim, cols, num_slots, cap, q_scale, floor_, head_stride};
  const dim3 grid((vdim + cols - 1) / cols, heads, num_seqs);
  launch_dependent(matrix_memory_scan_kernel, grid, SCAN_THREADS, smem, stream, a);
  return shrike_launch_status();
}

SHRIKE_API int shrike_matrix_memory_out(const float* numerator, const float* denominator, const float* fused, int partials,
                                        long long stride, int total, int gate_first, const float* weight, float eps, void* out,
                                        int dtype, int n, int heads, int vdim, cudaStream_t stream) {
  if (n <= 0) return SHRIKE_OK;
  if (heads < 1 || vdim < 1 || partials < 1 || gate_first < 0 || gate_first + heads * vdim > total) return SHRIKE_BAD_ARGUMENT;
  MemoryOutArgs a = {numerator, denominator, fused, stride, partials, total, gate_first, weight, eps, out, n, heads, vdim};
  const long long work = static_cast<long long>(n) * heads;
  const unsigned blocks = static_cast<unsigned>((work + PREP_WARPS - 1) / PREP_WARPS);
  if (dtype == SHRIKE_F32) launch_dependent(matrix_memory_out_kernel<float>, blocks, PREP_WARPS * 32, 0, stream, a);
  else if (dtype == SHRIKE_BF16) launch_dependent(matrix_memory_out_kernel<__nv_bfloat16>, blocks, PREP_WARPS * 32, 0, stream, a);
  else return SHRIKE_BAD_ARGUMENT;
  return shrike_launch_status();
}

// weights [N][columns], columns = experts (+ 1 when there is a shared expert: its gate, sigmoid(shared_gate . x), or 1
// when shared_gate is null).
// `sigmoid_scores`: an expert's score is the sigmoid of its logit instead of its softmax share; `renormalise` 0: the
// chosen experts keep their scores as they are.
SHRIKE_API int shrike_route_top_scores(const void* x, int dtype, const float* router, const float* shared_gate, float* weights, int n,
                                       int width, int experts, int top, int columns, float renorm_eps, int sigmoid_scores,
                                       int renormalise, cudaStream_t stream) {
  if (n <= 0) return SHRIKE_OK;
  if (experts < 1 || top < 1 || top > experts || experts > 1024 || (columns != experts && columns != experts + 1)) return SHRIKE_BAD_ARGUMENT;
  const unsigned blocks = static_cast<unsigned>(n);
  const size_t smem = static_cast<size_t>(ROUTE_WARPS) * (experts + 1) * sizeof(float);
  if (dtype == SHRIKE_F32)
    launch_dependent(route_top_kernel<float>, blocks, ROUTE_WARPS * 32, smem, stream, static_cast<const float*>(x), router,
                     shared_gate, weights, n, width, experts, top, columns, renorm_eps, sigmoid_scores, renormalise);
  else if (dtype == SHRIKE_BF16)
    launch_dependent(route_top_kernel<__nv_bfloat16>, blocks, ROUTE_WARPS * 32, smem, stream, static_cast<const __nv_bfloat16*>(x),
                     router, shared_gate, weights, n, width, experts, top, columns, renorm_eps, sigmoid_scores, renormalise);
  else return SHRIKE_BAD_ARGUMENT;
  return shrike_launch_status();
}

SHRIKE_API int shrike_route_top(const void* x, int dtype, const float* router, const float* shared_gate, float* weights, int n,
                                int width, int experts, int top, int columns, float renorm_eps, cudaStream_t stream) {
  return shrike_route_top_scores(x, dtype, router, shared_gate, weights, n, width, experts, top, columns, renorm_eps, 0, 1, stream);
}

// `weight_input` 1: an expert's weight multiplies its input, out = act(w gate) * (w up), instead of its output.
SHRIKE_API int shrike_act_mul_blocks_at(const void* gate_up, const float* weights, void* out, int dtype, int n, int inter, int experts,
                                        int each, int columns, int act, float limit, int weight_input, cudaStream_t stream) {
  if (n <= 0) return SHRIKE_OK;
  if (inter < 1 || experts < 1 || each < 1 || experts * each > inter || !known_activation(act)) return SHRIKE_BAD_ARGUMENT;
  if (experts * each < inter && columns != experts + 1) return SHRIKE_BAD_ARGUMENT;
  const int wide_f32 = 4, wide_bf16 = 8;
  const bool aligned = (reinterpret_cast<uintptr_t>(gate_up) | reinterpret_cast<uintptr_t>(out)) % 16 == 0;
  if (dtype == SHRIKE_F32) {
    const bool vec = aligned && inter % wide_f32 == 0 && each % wide_f32 == 0;
    const int groups = vec ? inter / wide_f32 : inter;
    const dim3 grid(max(1, min(64, (groups + 255) / 256)), max(1, min(n, 65535)));
    if (vec)
      launch_dependent(act_mul_blocks_kernel<float, 4>, grid, 256, 0, stream, static_cast<const float*>(gate_up), weights,
                       static_cast<float*>(out), n, inter, experts, each, columns, act, limit, weight_input);
    else
      launch_dependent(act_mul_blocks_kernel<float, 1>, grid, 256, 0, stream, static_cast<const float*>(gate_up), weights,
                       static_cast<float*>(out), n, inter, experts, each, columns, act, limit, weight_input);
  } else if (dtype == SHRIKE_BF16) {
    const bool vec = aligned && inter % wide_bf16 == 0 && each % wide_bf16 == 0;
    const int groups = vec ? inter / wide_bf16 : inter;
    const dim3 grid(max(1, min(64, (groups + 255) / 256)), max(1, min(n, 65535)));
    if (vec)
      launch_dependent(act_mul_blocks_kernel<__nv_bfloat16, 8>, grid, 256, 0, stream, static_cast<const __nv_bfloat16*>(gate_up),
                       weights, static_cast<__nv_bfloat16*>(out), n, inter, experts, each, columns, act, limit, weight_input);
    else
      launch_dependent(act_mul_blocks_kernel<__nv_bfloat16, 1>, grid, 256, 0, stream, static_cast<const __nv_bfloat16*>(gate_up),
                       weights, static_cast<__nv_bfloat16*>(out), n, inter, experts, each, columns, act, limit, weight_input);
  } else return SHRIKE_BAD_ARGUMENT;
  return shrike_launch_status();
}

SHRIKE_API int shrike_act_mul_blocks(const void* gate_up, const float* weights, void* out, int dtype, int n, int inter, int experts,
                                     int each, int columns, int act, float limit, cudaStream_t stream) {
  return shrike_act_mul_blocks_at(gate_up, weights, out, dtype, n, inter, experts, each, columns, act, limit, 0, stream);
}
