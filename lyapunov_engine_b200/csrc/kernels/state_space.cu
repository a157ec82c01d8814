// Diagonal state-space recurrences (selective scans) over the step's tokens,
// request by request, from each request's state row and back into it.
//
// Every row r (a channel) keeps N numbers of state.  Per token:
//
//   dt    = softplus(dt_raw + dt_bias)                       (one per row, or one per head of P rows)
//   S[n] <- exp(dt * A[n]) * S[n] + dt * x * B[n]            A = -exp(A_log): per (row, n), or one per head
//   y     = sum_n S[n] * C[n] + D * x                        D per row or per head
//   out   = y * silu(z) * out_scale                          (z: the gate's rows; null: out = y * out_scale)
//
// B and C are shared by the rows of a group (`rows_per_group` consecutive
// rows).  Both forms of the design family run here: one decay per head and
// step sizes per head (state-space duality), or decays per row and state and
// step sizes per row (the selective scan).  Step sizes, decays (le::exp_unbiased:
// they multiply up over the whole sequence), the recurrence, the sum and the gate are 32-bit; x, B, C, dt_raw and z come in
// the activations' type; the state is float32 [state rows, rows, N].
//
// A block takes one request and ROWS consecutive rows of one group; a row has
// LANES threads, each with every LANES-th entry of the row's state in
// registers.  The request's tokens pass in tiles of TILE through shared memory
// (B and C of the group, x, step sizes and gates of the block's rows); within
// a tile the threads run without meeting, the tile's outputs leave together.
// One launch serves every cut of the work: a request brings its next q_len
// tokens, 1 for a decoded token.  Requests without a state row (slot < 0,
// padding of a fixed-shape step) are skipped; their output rows are zeroed.
#include "common.cuh"

namespace {

constexpr int SSM_THREADS = 256;
constexpr int SSM_TILE = 16;
constexpr int SSM_GROUP = 1;      // tokens whose instructions overlap (SSM_TILE is a multiple); more than 1 did not pay
constexpr int SSM_AHEAD = 8;      // loads a staging thread has in flight

__device__ __forceinline__ float softplus_f32(float v) { return v > 20.0f ? v : log1pf(expf(v)); }

struct SsmArgs {
  const void *x; int64_t x_stride;
  const void *bc; int64_t bc_stride; int b_col, c_col;     // B at b_col + group * N, C at c_col + group * N
  const void *dt; int64_t dt_stride;
  const void *z; int64_t z_stride;
  void *out; int64_t out_stride;
  const float *dt_bias, *a_log, *d_skip;
  float *state; int num_state_rows;
  const int32_t *state_slots, *cu_q;
  int rows, n_state, rows_per_head, rows_per_group, rows_per_block;
  float out_scale;
};

template <typename T, typename TO, int NPER, int LANES, bool PER_ROW>
__global__ void __launch_bounds__(SSM_THREADS)
ssm_scan_kernel(SsmArgs p) {
  extern __shared__ __align__(16) float ssm_smem[];
  const int N = p.n_state, ROWS = p.rows_per_block;
  float *s_b = ssm_smem;                       // [TILE][N]
  float *s_c = s_b + SSM_TILE * N;             // [TILE][N]
  float *s_x = s_c + SSM_TILE * N;             // [TILE][ROWS]
  float *s_dt = s_x + SSM_TILE * ROWS;         // [TILE][ROWS]
  float *s_y = s_dt + SSM_TILE * ROWS;         // [TILE][ROWS]
  float *s_dec = s_y + SSM_TILE * ROWS;        // [TILE][ROWS]: the decay of a row's head (one decay per head only)
  le::let_successor_start();
  const int b = blockIdx.y;
  const int row0 = blockIdx.x * ROWS;
  const int r = threadIdx.x / LANES, lane = threadIdx.x % LANES;
  const int row = row0 + r;
  const bool active = r < ROWS && row < p.rows;
  const int head = row / p.rows_per_head;
  const int group = row0 / p.rows_per_group;
  const int first = p.cu_q[b], q_len = p.cu_q[b + 1] - first;
  const int slot = p.state_slots[b];
  const bool has_state = slot >= 0 && slot < p.num_state_rows;
  const int threads = ROWS * LANES;

  // this thread's decay rates and the row's skip factor: parameters, not the predecessor's output
  float a[NPER];
  float d_skip = 0.0f;
  if (active) {
    d_skip = p.d_skip != nullptr ? p.d_skip[PER_ROW ? row : head] : 0.0f;
#pragma unroll
    for (int j = 0; j < NPER; ++j) {
      const int n = lane + LANES * j;
      if constexpr (PER_ROW) a[j] = n < N ? -expf(p.a_log[static_cast<int64_t>(row) * N + n]) : 0.0f;
      else a[j] = -expf(p.a_log[head]);
    }
  }
  float S[NPER];
#pragma unroll
  for (int j = 0; j < NPER; ++j) S[j] = 0.0f;
  float *mine = has_state && active ? p.state + (static_cast<int64_t>(slot) * p.rows + row) * N : nullptr;
  le::wait_for_predecessor();
  if (mine != nullptr) {
#pragma unroll
    for (int j = 0; j < NPER; ++j) {
      const int n = lane + LANES * j;
      if (n < N) S[j] = mine[n];
    }
  }
  const T *xs = static_cast<const T *>(p.x);
  const T *bcs = static_cast<const T *>(p.bc);
  const T *dts = static_cast<const T *>(p.dt);
  const T *zs = static_cast<const T *>(p.z);
  TO *outs = static_cast<TO *>(p.out);

  for (int t0 = 0; t0 < q_len; t0 += SSM_TILE) {
    const int tile = min(SSM_TILE, q_len - t0);
    __syncthreads();                                   // the tile before is stored
    const int padded = (tile + SSM_GROUP - 1) / SSM_GROUP * SSM_GROUP;       // whole groups: zeros behind the tile's tokens
    // B and C of the tile's tokens (every block of a group stages the same ones, so this must be cheap): in 16-byte
    // pieces where the layout allows, else value by value with SSM_AHEAD loads in flight per thread (a load and its
    // store one after the other would wait out the memory's latency once per value)
    constexpr int PIECE = le::Piece16<T>::COUNT;
    const bool pieces = N % PIECE == 0 && p.b_col % PIECE == 0 && p.c_col % PIECE == 0 && p.bc_stride % PIECE == 0 &&
                        (reinterpret_cast<uintptr_t>(bcs) & 15) == 0;
    if (pieces) {
      const int per_token = N / PIECE;
      for (int i = threadIdx.x; i < padded * per_token; i += threads) {
        const int t = i / per_token, n = (i - t * per_token) * PIECE;
        float bv[PIECE], cv[PIECE];
        if (t < tile) {
          const T *src = bcs + static_cast<int64_t>(first + t0 + t) * p.bc_stride + group * N + n;
          le::load_piece16<T>(bv, src + p.b_col);
          le::load_piece16<T>(cv, src + p.c_col);
        } else {
#pragma unroll
          for (int v = 0; v < PIECE; ++v) bv[v] = cv[v] = 0.0f;
        }
#pragma unroll
        for (int v = 0; v < PIECE; v += 4) {
          *reinterpret_cast<float4 *>(s_b + t * N + n + v) = make_float4(bv[v], bv[v + 1], bv[v + 2], bv[v + 3]);
          *reinterpret_cast<float4 *>(s_c + t * N + n + v) = make_float4(cv[v], cv[v + 1], cv[v + 2], cv[v + 3]);
        }
      }
    } else {
      for (int base = threadIdx.x; base < padded * N; base += threads * SSM_AHEAD) {
        float bv[SSM_AHEAD], cv[SSM_AHEAD];
#pragma unroll
        for (int u = 0; u < SSM_AHEAD; ++u) {
          const int i = base + u * threads;
          const int t = i / N, n = i - t * N;
          bv[u] = cv[u] = 0.0f;
          if (i < padded * N && t < tile) {
            const T *src = bcs + static_cast<int64_t>(first + t0 + t) * p.bc_stride + group * N + n;
            bv[u] = le::to_f32(src[p.b_col]), cv[u] = le::to_f32(src[p.c_col]);
          }
        }
#pragma unroll
        for (int u = 0; u < SSM_AHEAD; ++u) {
          const int i = base + u * threads;
          if (i < padded * N) s_b[i] = bv[u], s_c[i] = cv[u];
        }
      }
    }
    for (int base = threadIdx.x; base < padded * ROWS; base += threads * SSM_AHEAD) {
      float xs_[SSM_AHEAD], ds_[SSM_AHEAD];
      int di_[SSM_AHEAD];
#pragma unroll
      for (int u = 0; u < SSM_AHEAD; ++u) {
        const int i = base + u * threads;
        const int t = i / ROWS, rr = i - t * ROWS;
        const int rw = row0 + rr;
        xs_[u] = 0.0f, ds_[u] = -INFINITY, di_[u] = -1;
        if (i < padded * ROWS && rw < p.rows && t < tile) {
          const int64_t tok = first + t0 + t;
          xs_[u] = le::to_f32(xs[tok * p.x_stride + rw]);
          di_[u] = PER_ROW ? rw : rw / p.rows_per_head;
          ds_[u] = le::to_f32(dts[tok * p.dt_stride + di_[u]]);
        }
      }
#pragma unroll
      for (int u = 0; u < SSM_AHEAD; ++u) {
        const int i = base + u * threads;
        if (i < padded * ROWS) {
          const float step = di_[u] >= 0 ? softplus_f32(ds_[u] + p.dt_bias[di_[u]]) : 0.0f;
          s_x[i] = xs_[u];
          s_dt[i] = step;
          // (one decay per head: made once per row and token here, not by every lane of the row)
          if constexpr (!PER_ROW) s_dec[i] = di_[u] >= 0 ? le::exp_unbiased(-step * expf(p.a_log[di_[u]])) : 1.0f;
        }
      }
    }
    __syncthreads();
    if (active && has_state) {
      // Tokens in groups of SSM_GROUP: the state's chain runs through them one after the other, but each token's
      // decays, products and the reduction of its sum over the lanes depend on nothing of the others, so the
      // instructions of a group overlap (a token by itself waits out the latencies of its shuffles and exponentials).
      // A tile's rows beyond its tokens hold zeros: a step size of zero leaves the state as it is.
      for (int t = 0; t < tile; t += SSM_GROUP) {
        float dv[SSM_GROUP], dx[SSM_GROUP], xv[SSM_GROUP], acc[SSM_GROUP], decay_all[SSM_GROUP];
#pragma unroll
        for (int u = 0; u < SSM_GROUP; ++u) {
          dv[u] = s_dt[(t + u) * ROWS + r], xv[u] = s_x[(t + u) * ROWS + r];
          dx[u] = dv[u] * xv[u];
          acc[u] = 0.0f;
          decay_all[u] = PER_ROW ? 0.0f : s_dec[(t + u) * ROWS + r];
        }
        const float *b_at = s_b + t * N + lane, *c_at = s_c + t * N + lane;     // (entry j lies LANES * j further: a constant)
#pragma unroll
        for (int j = 0; j < NPER; ++j) {
          const int n = lane + LANES * j;
          if (n < N) {
            float decay[SSM_GROUP];
#pragma unroll
            for (int u = 0; u < SSM_GROUP; ++u) decay[u] = PER_ROW ? le::exp_unbiased(dv[u] * a[j]) : decay_all[u];
#pragma unroll
            for (int u = 0; u < SSM_GROUP; ++u) {
              S[j] = fmaf(decay[u], S[j], dx[u] * b_at[u * N + LANES * j]);
              acc[u] = fmaf(S[j], c_at[u * N + LANES * j], acc[u]);
            }
          }
        }
#pragma unroll
        for (int o = LANES / 2; o > 0; o >>= 1) {
#pragma unroll
          for (int u = 0; u < SSM_GROUP; ++u) acc[u] += __shfl_xor_sync(0xffffffffu, acc[u], o);
        }
        if (lane == 0) {
#pragma unroll
          for (int u = 0; u < SSM_GROUP; ++u) s_y[(t + u) * ROWS + r] = fmaf(d_skip, xv[u], acc[u]);
        }
      }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < tile * ROWS; i += threads) {
      const int t = i / ROWS, rr = i - t * ROWS;
      const int64_t tok = first + t0 + t;
      const int rw = row0 + rr;
      if (rw >= p.rows) continue;
      float y = has_state ? s_y[t * ROWS + rr] : 0.0f;
      if (zs != nullptr) {
        const float g = le::to_f32(zs[tok * p.z_stride + rw]);
        y *= g / (1.0f + expf(-g));
      }
      outs[tok * p.out_stride + rw] = le::from_f32<TO>(y * p.out_scale);
    }
  }
  if (mine != nullptr) {
#pragma unroll
    for (int j = 0; j < NPER; ++j) {
      const int n = lane + LANES * j;
      if (n < N) mine[n] = S[j];
    }
  }
}

template <typename T, typename TO, int NPER, int LANES>
int launch_ssm(const SsmArgs &p, int per_row, int num_requests, cudaStream_t stream) {
  const int rows_per_block = p.rows_per_block;
  const dim3 grid((p.rows + rows_per_block - 1) / rows_per_block, num_requests);
  const size_t smem = sizeof(float) * (2 * SSM_TILE * p.n_state + 4 * SSM_TILE * rows_per_block);
  if (smem > 200 * 1024) return le::invalid("le_ssm_scan: %d numbers of state per row do not fit a block's shared memory", p.n_state);
  const dim3 block(rows_per_block * LANES);
  auto kernel = per_row ? ssm_scan_kernel<T, TO, NPER, LANES, true> : ssm_scan_kernel<T, TO, NPER, LANES, false>;
  if (smem > 48 * 1024) {
    static size_t raised[2] = {0, 0};            // per form and process: the most asked for so far
    if (smem > raised[per_row ? 1 : 0]) {
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
      if (e != cudaSuccess) return le::invalid("le_ssm_scan: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
      raised[per_row ? 1 : 0] = smem;
    }
  }
  return le::launch_chained(kernel, grid, block, smem, stream, p);
}

template <typename T, typename TO, int LANES>
int launch_ssm_lanes(const SsmArgs &p, int per_row, int num_requests, cudaStream_t stream) {
  const int nper = (p.n_state + LANES - 1) / LANES;
  switch (nper) {
    case 1: case 2: return launch_ssm<T, TO, 2, LANES>(p, per_row, num_requests, stream);
    case 3: case 4: return launch_ssm<T, TO, 4, LANES>(p, per_row, num_requests, stream);
    case 5: case 6: return launch_ssm<T, TO, 6, LANES>(p, per_row, num_requests, stream);
    case 7: case 8: return launch_ssm<T, TO, 8, LANES>(p, per_row, num_requests, stream);
    default: break;
  }
  if constexpr (LANES == 32) {
    if (nper <= 16) return launch_ssm<T, TO, 16, LANES>(p, per_row, num_requests, stream);
  }
  return le::invalid("le_ssm_scan: at most %d numbers of state per row, got %d", 16 * LANES, p.n_state);
}

}  // namespace

// How many threads share a row's state of `n_state` numbers.  One decay per head: up to 8 entries a thread (the
// block's rows share staged B and C, and many rows a block amortise that staging).  A decay per row and state: an
// exponential per entry is the work, and a request's rows times these lanes are all the threads a prompt has, so
// one or two entries a thread (`spread`; not in a step of single tokens, which only moves the states through).
static int ssm_lanes(int n_state, int spread) {
  int lanes = 4;
  while (lanes < 32 && (n_state + lanes - 1) / lanes > (spread ? 1 : 8)) lanes *= 2;
  return lanes;
}

// The rows a block takes: a divisor of a group's rows (a block's rows share B and C) that fits its threads.  One
// decay per head: the most that fit.  A decay per row and state: the most that still leave two blocks for every
// multiprocessor (a block of a warp at least).
static int ssm_rows_per_block(int n_state, int rows, int rows_per_group, int spread, int num_requests) {
  const int lanes = ssm_lanes(n_state, spread);
  const int most = SSM_THREADS / lanes;
  int best = 1, roomy = 0;
  for (int c = 1; c <= most; ++c) {
    if (rows_per_group % c) continue;
    best = c;
    if (static_cast<int64_t>(rows / c) * num_requests >= 296 || c * lanes <= 32) roomy = c;
  }
  return spread && roomy > 0 ? roomy : best;
}

// x [T, rows] (row stride x_stride), bc: rows holding B [groups, n_state] at column b_col and C at c_col, dt
// [T, rows or heads], z [T, rows] or null: all of type `dtype`; out [T, rows] of type `out_dtype`.  per_row 1: dt,
// dt_bias and d_skip have one entry per row and a_log is [rows, n_state]; 0: one per head of rows_per_head rows.
// state: float32 [num_state_rows, rows, n_state]; request b (tokens cu_q[b] .. cu_q[b + 1]) owns row state_slots[b];
// num_tokens: the step's tokens in all (it only chooses the launch's shape).
LE_API int le_ssm_scan(void *out, int out_dtype, int64_t out_stride, const void *x, int64_t x_stride, const void *bc,
                       int64_t bc_stride, int b_col, int c_col, const void *dt, int64_t dt_stride, const void *z,
                       int64_t z_stride, int dtype, const float *dt_bias, const float *a_log, const float *d_skip,
                       float *state, int num_state_rows, const int32_t *state_slots, const int32_t *cu_q, int num_requests,
                       int num_tokens, int rows, int n_state, int rows_per_head, int rows_per_group, int per_row,
                       float out_scale, cudaStream_t stream) {
  if (num_requests <= 0 || rows <= 0) return 0;
  if (num_requests > 65535) return le::invalid("le_ssm_scan: too many requests for one launch");
  if (n_state < 1 || rows_per_head < 1 || rows_per_group < 1 || rows % rows_per_group || rows_per_group % rows_per_head)
    return le::invalid("le_ssm_scan: %d rows in heads of %d and groups of %d", rows, rows_per_head, rows_per_group);
  SsmArgs p;
  p.x = x, p.x_stride = x_stride, p.bc = bc, p.bc_stride = bc_stride, p.b_col = b_col, p.c_col = c_col;
  p.dt = dt, p.dt_stride = dt_stride, p.z = z, p.z_stride = z_stride, p.out = out, p.out_stride = out_stride;
  p.dt_bias = dt_bias, p.a_log = a_log, p.d_skip = d_skip, p.state = state, p.num_state_rows = num_state_rows;
  p.state_slots = state_slots, p.cu_q = cu_q, p.rows = rows, p.n_state = n_state, p.rows_per_head = rows_per_head;
  p.rows_per_group = rows_per_group, p.out_scale = out_scale;
  const int spread = per_row && num_tokens > num_requests;
  p.rows_per_block = ssm_rows_per_block(n_state, rows, rows_per_group, spread, num_requests);
  const int lanes = ssm_lanes(n_state, spread);
#define LE_SSM(T, TO)                                                                              \
  do {                                                                                             \
    if (lanes == 4) return launch_ssm_lanes<T, TO, 4>(p, per_row, num_requests, stream);           \
    if (lanes == 8) return launch_ssm_lanes<T, TO, 8>(p, per_row, num_requests, stream);           \
    if (lanes == 16) return launch_ssm_lanes<T, TO, 16>(p, per_row, num_requests, stream);         \
    return launch_ssm_lanes<T, TO, 32>(p, per_row, num_requests, stream);                          \
  } while (0)
  if (dtype == LE_F32 && out_dtype == LE_F32) LE_SSM(float, float);
  if (dtype == LE_BF16 && out_dtype == LE_F32) LE_SSM(__nv_bfloat16, float);
  if (dtype == LE_BF16 && out_dtype == LE_BF16) LE_SSM(__nv_bfloat16, __nv_bfloat16);
#undef LE_SSM
  return le::invalid("le_ssm_scan: no form for input type %d and output type %d", dtype, out_dtype);
}
