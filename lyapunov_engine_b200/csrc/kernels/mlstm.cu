// The matrix memory of the mLSTM over the step's tokens, request by request,
// from each request's state row and back into it.
//
// Per head, with q (already times its scale), k [dim], v [vdim] and two gate
// pre-activations a_i, a_f per token:
//
//   i = cap * tanh((a_i + b_i) / cap)              f = logsigmoid(cap * tanh((a_f + b_f) / cap))
//   m' = max(f + m, i)                             (m starts at 0)
//   S <- exp(f + m - m') S + exp(i - m') k v^T     n <- exp(f + m - m') n + exp(i - m') k
//   o  = S^T q / (max(|n . q|, exp(-m')) + 1e-6)
//
// All of it 32-bit; q, k, v and the pre-activations come in the activations'
// type.
//
// A block takes one request, one head and ROWS of the vdim columns of S; a
// column has LANES threads, each with every LANES-th entry in registers.  One
// more group of LANES threads carries n, and the block its own m: every block
// needs n . q and the gates, so every block keeps a copy of n and m beside its
// columns and no block reads what another writes.  State per request and
// head, float32 [vdim / ROWS, ROWS + 2, dim]: of a block's part, row r < ROWS
// is column r of its columns of S (a thread's entries are consecutive), row
// ROWS is n and the first entry of row ROWS + 1 is m (le_mlstm_rows() says
// what ROWS is for a head's sizes).  Tokens pass in tiles through
// shared memory; the gates of a tile are made by the first warp: the
// pre-activations' functions side by side, the running maximum by one thread
// (an addition and a maximum per token), the three exponentials side by side.
// Within a tile the threads run without meeting; numerators and n . q are
// left in shared memory and divided as the tile is stored.
#include "common.cuh"

namespace {

constexpr int ML_TILE = 16;
constexpr int ML_GROUP = 1;        // tokens whose instructions overlap; more than 1 did not pay
constexpr int ML_AHEAD = 8;        // loads a staging thread has in flight
constexpr int ML_MAX_THREADS = 256;

__device__ __forceinline__ float log_sigmoid_f32(float x) {
  // -softplus(-x), without overflow on either side
  return x >= 0.0f ? -log1pf(expf(-x)) : x - log1pf(expf(x));
}

struct MlstmArgs {
  float *out; int64_t out_stride;                 // [T, heads * vdim] float32
  const void *qkv; int64_t qkv_stride; int q_col, k_col, v_col, i_col, f_col;
  const float *i_bias, *f_bias;
  float *state; int num_state_rows;
  const int32_t *state_slots, *cu_q;
  int heads, dim, vdim, rows_per_block;
  float cap, q_scale;
};

template <typename T, int NPER, int LANES>
__global__ void __launch_bounds__(ML_MAX_THREADS)
mlstm_scan_kernel(MlstmArgs p) {
  extern __shared__ __align__(16) float ml_smem[];
  const int D = p.dim, ROWS = p.rows_per_block;
  float *s_q = ml_smem;                          // [TILE][D]
  float *s_k = s_q + ML_TILE * D;                // [TILE][D]
  float *s_v = s_k + ML_TILE * D;                // [TILE][ROWS]
  float *s_num = s_v + ML_TILE * ROWS;           // [TILE][ROWS]
  float *s_gate = s_num + ML_TILE * ROWS;        // [6][TILE]: i, f, keep, take, floor, n . q
  __shared__ float s_m;                          // the running maximum between tiles
  le::let_successor_start();
  const int b = blockIdx.z, head = blockIdx.y, e0 = blockIdx.x * ROWS;
  const int r = threadIdx.x / LANES, lane = threadIdx.x % LANES;
  const bool is_n = r == ROWS;                   // the group that carries n
  const int first = p.cu_q[b], q_len = p.cu_q[b + 1] - first;
  const int slot = p.state_slots[b];
  const bool has_state = slot >= 0 && slot < p.num_state_rows;
  const int threads = (ROWS + 1) * LANES;
  // this block's part of the head's state: its columns, its copy of n, its copy of m
  float *head_state = has_state ? p.state + ((static_cast<int64_t>(slot) * p.heads + head) * gridDim.x + blockIdx.x) * (ROWS + 2) * D
                                : nullptr;
  float *mine = head_state != nullptr ? head_state + static_cast<int64_t>(r) * D : nullptr;
  const float bias_i = p.i_bias[head], bias_f = p.f_bias[head];
  float S[NPER];
#pragma unroll
  for (int j = 0; j < NPER; ++j) S[j] = 0.0f;
  le::wait_for_predecessor();
  if (mine != nullptr) {
#pragma unroll
    for (int j = 0; j < NPER; ++j) {
      const int d = lane + LANES * j;
      if (d < D) S[j] = mine[d];
    }
  }
  if (threadIdx.x == 0) s_m = head_state != nullptr ? head_state[static_cast<int64_t>(ROWS + 1) * D] : 0.0f;
  const T *rows = static_cast<const T *>(p.qkv);

  for (int t0 = 0; t0 < q_len; t0 += ML_TILE) {
    const int tile = min(ML_TILE, q_len - t0);
    __syncthreads();                               // the tile before is stored
    const int gate_threads = min(32, threads);
    if (threadIdx.x < gate_threads) {
      // the tile's gates, by the first warp
      for (int t = threadIdx.x; t < tile; t += gate_threads) {
        const T *row = rows + static_cast<int64_t>(first + t0 + t) * p.qkv_stride;
        s_gate[0 * ML_TILE + t] = p.cap * tanhf((le::to_f32(row[p.i_col + head]) + bias_i) / p.cap);
        s_gate[1 * ML_TILE + t] = log_sigmoid_f32(p.cap * tanhf((le::to_f32(row[p.f_col + head]) + bias_f) / p.cap));
      }
      __syncwarp();
      if (threadIdx.x == 0) {
        float m = s_m;
        for (int u = 0; u < tile; ++u) {
          const float m_new = fmaxf(s_gate[1 * ML_TILE + u] + m, s_gate[0 * ML_TILE + u]);
          s_gate[2 * ML_TILE + u] = m;            // (the maximum before the token, for the next phase)
          s_gate[4 * ML_TILE + u] = m_new;
          m = m_new;
        }
        s_m = m;
      }
      __syncwarp();
      for (int t = threadIdx.x; t < tile; t += gate_threads) {
        const float m_old = s_gate[2 * ML_TILE + t], m_new = s_gate[4 * ML_TILE + t];
        // (factors that multiply up over the sequence: the exponential that does not lean to one side)
        s_gate[2 * ML_TILE + t] = le::exp_unbiased(s_gate[1 * ML_TILE + t] + m_old - m_new);
        s_gate[3 * ML_TILE + t] = le::exp_unbiased(s_gate[0 * ML_TILE + t] - m_new);
        s_gate[4 * ML_TILE + t] = le::exp_unbiased(-m_new);
      }
    }
    // q and k of the tile's tokens (every block of a head stages the same ones, so this must be cheap): in 16-byte
    // pieces where the layout allows, else value by value with ML_AHEAD loads in flight per thread
    constexpr int PIECE = le::Piece16<T>::COUNT;
    const bool pieces = D % PIECE == 0 && p.q_col % PIECE == 0 && p.k_col % PIECE == 0 && p.qkv_stride % PIECE == 0 &&
                        (reinterpret_cast<uintptr_t>(rows) & 15) == 0;
    if (pieces) {
      const int per_token = D / PIECE;
      for (int i = threadIdx.x; i < tile * per_token; i += threads) {
        const int t = i / per_token, d = (i - t * per_token) * PIECE;
        const T *row = rows + static_cast<int64_t>(first + t0 + t) * p.qkv_stride + head * D + d;
        float qv[PIECE], kv[PIECE];
        le::load_piece16<T>(qv, row + p.q_col);
        le::load_piece16<T>(kv, row + p.k_col);
#pragma unroll
        for (int v = 0; v < PIECE; v += 4) {
          *reinterpret_cast<float4 *>(s_q + t * D + d + v) =
              make_float4(qv[v] * p.q_scale, qv[v + 1] * p.q_scale, qv[v + 2] * p.q_scale, qv[v + 3] * p.q_scale);
          *reinterpret_cast<float4 *>(s_k + t * D + d + v) = make_float4(kv[v], kv[v + 1], kv[v + 2], kv[v + 3]);
        }
      }
    } else {
      for (int base = threadIdx.x; base < tile * D; base += threads * ML_AHEAD) {
        float qv[ML_AHEAD], kv[ML_AHEAD];
#pragma unroll
        for (int u = 0; u < ML_AHEAD; ++u) {
          const int i = base + u * threads;
          qv[u] = kv[u] = 0.0f;
          if (i < tile * D) {
            const int t = i / D, d = i - t * D;
            const T *row = rows + static_cast<int64_t>(first + t0 + t) * p.qkv_stride + head * D + d;
            qv[u] = le::to_f32(row[p.q_col]), kv[u] = le::to_f32(row[p.k_col]);
          }
        }
#pragma unroll
        for (int u = 0; u < ML_AHEAD; ++u) {
          const int i = base + u * threads;
          if (i < tile * D) s_q[i] = qv[u] * p.q_scale, s_k[i] = kv[u];
        }
      }
    }
    for (int i = threadIdx.x; i < tile * ROWS; i += threads) {
      const int t = i / ROWS, rr = i - t * ROWS;
      s_v[t * ROWS + rr] = le::to_f32(rows[static_cast<int64_t>(first + t0 + t) * p.qkv_stride + p.v_col + head * p.vdim + e0 + rr]);
    }
    __syncthreads();
    if (has_state) {
      // Tokens in groups of ML_GROUP: the state's chain runs through them one after the other, but each token's
      // products and the reduction of its sum over the lanes depend on nothing of the others, so a group's
      // instructions overlap.  A tile's rows beyond its tokens keep everything (factor 1) and take nothing (0).
      for (int t = 0; t < tile; t += ML_GROUP) {
        float keep[ML_GROUP], in[ML_GROUP], acc[ML_GROUP];
#pragma unroll
        for (int u = 0; u < ML_GROUP; ++u) {
          const bool live = t + u < tile;
          keep[u] = live ? s_gate[2 * ML_TILE + t + u] : 1.0f;
          in[u] = live ? s_gate[3 * ML_TILE + t + u] * (is_n ? 1.0f : s_v[(t + u) * ROWS + r]) : 0.0f;
          acc[u] = 0.0f;
        }
#pragma unroll
        for (int j = 0; j < NPER; ++j) {
          const int d = lane + LANES * j;
          if (d < D) {
#pragma unroll
            for (int u = 0; u < ML_GROUP; ++u) {
              const int tt = min(t + u, tile - 1);
              S[j] = fmaf(keep[u], S[j], in[u] * s_k[tt * D + d]);
              acc[u] = fmaf(S[j], s_q[tt * D + d], acc[u]);
            }
          }
        }
#pragma unroll
        for (int o = LANES / 2; o > 0; o >>= 1) {
#pragma unroll
          for (int u = 0; u < ML_GROUP; ++u) acc[u] += __shfl_xor_sync(0xffffffffu, acc[u], o);
        }
        if (lane == 0) {
#pragma unroll
          for (int u = 0; u < ML_GROUP; ++u) {
            if (t + u < tile) {
              if (is_n) s_gate[5 * ML_TILE + t + u] = acc[u];
              else s_num[(t + u) * ROWS + r] = acc[u];
            }
          }
        }
      }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < tile * ROWS; i += threads) {
      const int t = i / ROWS, rr = i - t * ROWS;
      float o = 0.0f;
      if (has_state) o = s_num[t * ROWS + rr] / (fmaxf(fabsf(s_gate[5 * ML_TILE + t]), s_gate[4 * ML_TILE + t]) + 1e-6f);
      p.out[static_cast<int64_t>(first + t0 + t) * p.out_stride + head * p.vdim + e0 + rr] = o;
    }
  }
  if (mine != nullptr) {
#pragma unroll
    for (int j = 0; j < NPER; ++j) {
      const int d = lane + LANES * j;
      if (d < D) mine[d] = S[j];
    }
  }
  __syncthreads();
  if (threadIdx.x == 0 && head_state != nullptr) head_state[static_cast<int64_t>(ROWS + 1) * D] = s_m;
}

int ml_lanes(int dim) {
  int lanes = 4;
  while (lanes < 32 && (dim + lanes - 1) / lanes > 8) lanes *= 2;
  return lanes;
}

int ml_rows(int dim, int vdim) {
  const int most = ML_MAX_THREADS / ml_lanes(dim) - 1;
  int rows = 1;
  for (int c = 1; c <= most; ++c)
    if (vdim % c == 0) rows = c;
  return rows;
}

template <typename T, int NPER, int LANES>
int launch_mlstm(const MlstmArgs &p, int num_requests, cudaStream_t stream) {
  const dim3 grid(p.vdim / p.rows_per_block, p.heads, num_requests);
  const size_t smem = sizeof(float) * (2 * ML_TILE * p.dim + 2 * ML_TILE * p.rows_per_block + 6 * ML_TILE);
  if (smem > 200 * 1024) return le::invalid("le_mlstm_scan: heads of %d entries do not fit a block's shared memory", p.dim);
  if (smem > 48 * 1024) {
    static size_t raised = 0;                    // per form and process: the most asked for so far
    if (smem > raised) {
      cudaError_t e = cudaFuncSetAttribute(mlstm_scan_kernel<T, NPER, LANES>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
      if (e != cudaSuccess) return le::invalid("le_mlstm_scan: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
      raised = smem;
    }
  }
  return le::launch_chained(mlstm_scan_kernel<T, NPER, LANES>, grid, dim3((p.rows_per_block + 1) * LANES), smem, stream, p);
}

template <typename T, int LANES>
int launch_mlstm_lanes(const MlstmArgs &p, int num_requests, cudaStream_t stream) {
  const int nper = (p.dim + LANES - 1) / LANES;
  if (nper <= 2) return launch_mlstm<T, 2, LANES>(p, num_requests, stream);
  if (nper <= 4) return launch_mlstm<T, 4, LANES>(p, num_requests, stream);
  if (nper <= 6) return launch_mlstm<T, 6, LANES>(p, num_requests, stream);
  if (nper <= 8) return launch_mlstm<T, 8, LANES>(p, num_requests, stream);
  if constexpr (LANES == 32) {
    if (nper <= 16) return launch_mlstm<T, 16, LANES>(p, num_requests, stream);
  }
  return le::invalid("le_mlstm_scan: heads of at most %d entries, got %d", 16 * LANES, p.dim);
}

}  // namespace

// out: float32 [T, heads * vdim].  rows (`dtype`): per token q [heads, dim] at q_col, k at k_col, v [heads, vdim] at
// v_col and one pre-activation per head at i_col and at f_col.  state: float32 [num_state_rows, heads, vdim / R, R + 2,
// dim] with R = le_mlstm_rows(dim, vdim).
LE_API int le_mlstm_rows(int dim, int vdim) { return dim >= 1 && vdim >= 1 ? ml_rows(dim, vdim) : 0; }

LE_API int le_mlstm_scan(float *out, int64_t out_stride, const void *rows, int64_t row_stride, int q_col, int k_col, int v_col,
                         int i_col, int f_col, int dtype, const float *i_bias, const float *f_bias, float *state,
                         int num_state_rows, const int32_t *state_slots, const int32_t *cu_q, int num_requests, int heads,
                         int dim, int vdim, float cap, float q_scale, cudaStream_t stream) {
  if (num_requests <= 0) return 0;
  if (heads < 1 || dim < 1 || vdim < 1 || heads > 65535 || num_requests > 65535)
    return le::invalid("le_mlstm_scan: %d heads of %d x %d for %d requests", heads, dim, vdim, num_requests);
  if (!(cap > 0.0f)) return le::invalid("le_mlstm_scan: the gates' cap must be positive");
  MlstmArgs p;
  p.out = out, p.out_stride = out_stride, p.qkv = rows, p.qkv_stride = row_stride;
  p.q_col = q_col, p.k_col = k_col, p.v_col = v_col, p.i_col = i_col, p.f_col = f_col;
  p.i_bias = i_bias, p.f_bias = f_bias, p.state = state, p.num_state_rows = num_state_rows;
  p.state_slots = state_slots, p.cu_q = cu_q, p.heads = heads, p.dim = dim, p.vdim = vdim;
  p.rows_per_block = ml_rows(dim, vdim), p.cap = cap, p.q_scale = q_scale;
  const int lanes = ml_lanes(dim);
#define LE_ML(T)                                                                  \
  do {                                                                            \
    if (lanes == 4) return launch_mlstm_lanes<T, 4>(p, num_requests, stream);     \
    if (lanes == 8) return launch_mlstm_lanes<T, 8>(p, num_requests, stream);     \
    if (lanes == 16) return launch_mlstm_lanes<T, 16>(p, num_requests, stream);   \
    return launch_mlstm_lanes<T, 32>(p, num_requests, stream);                    \
  } while (0)
  if (dtype == LE_F32) LE_ML(float);
  if (dtype == LE_BF16) LE_ML(__nv_bfloat16);
#undef LE_ML
  return le::invalid("le_mlstm_scan: unknown dtype code %d", dtype);
}
