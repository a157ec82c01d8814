// Routed experts: the router, the grouping of (token, choice) pairs by expert,
// the products over those groups, and the weighted sum.
//
// route:   z = Wr h + b in 32 bits (Wr, b float32; h in the activations'
//          type), the `top` largest z (ties: the lower index), their weights
//          softmax over the chosen z only; and, where given, one more number
//          per token, sigmoid(sg . h), for a shared expert.  Two kernels: the
//          logits (blocks over tokens and over rows of the router), the choice.
// group:   pair p = t * top + j goes to expert id[p].  Counting sort in one
//          block: offsets per expert, the pairs in expert order, and a list of
//          row tiles (expert, first sorted slot, rows), each tile within one
//          expert.  The order of an expert's pairs is arbitrary; no result
//          depends on it, every row of a product is computed by itself.
// grouped: C[row] = A[src(row)] W[expert]^T over the tiles, FP32 pipes, inputs
//          float32 or bfloat16, sums in ascending k in float32.  Gated form:
//          W[expert] is [2 F, K] (gate rows, then up rows) and C = act(gate,
//          up), F wide.  Input rows are gathered through `src_of_slot` divided
//          by `src_div` (pairs -> tokens) or are the sorted slots themselves;
//          output rows go to the sorted slot or are scattered back to the pair
//          with the pair's weight as a factor (float32 output).  In the gated
//          form a pair's weight is the factor on the expert's input instead:
//          both products are multiplied by it, in 32 bits, before the activation.
// combine: out[t] = sum_j y[t * top + j] (+ gate[t] * shared[t]).
// Where experts have many rows each (prompt portions, bfloat16) the products run on the tcgen05 kernel of
// gemm_tc.cu in its grouped form instead: the grouping pads every expert's slots to whole tiles of 128, the rows of
// x are gathered into slot order, both products run over the sorted rows, and the weighted sum reads them back
// through each pair's slot.
#include "common.cuh"

namespace {

constexpr int TILE_M = 32;        // sorted slots per tile
constexpr int TILE_M_WIDE = 128;  // of the tensor-core kernel where experts have many rows each
constexpr int TILE_N = 64;   // output columns per block
constexpr int TILE_K = 32;

constexpr int ROUTE_WARPS = 16;
constexpr int ROUTE_SMEM_FLOATS = 16 * 1024;   // of the tokens' rows a block holds as float32

// Four consecutive activations in one access, as floats.
template <typename T> struct RoutePiece;
template <> struct RoutePiece<float> { using type = float4; };
template <> struct RoutePiece<__nv_bfloat16> { using type = uint2; };
__device__ __forceinline__ void unpack4(const float4 &a, float (&v)[4]) { v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; }
__device__ __forceinline__ void unpack4(const uint2 &raw, float (&v)[4]) {
  const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&raw);
  const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}

// Router logits.  A block takes NT tokens and RB rows of the router (the shared gate's row counts as one more): the
// tokens' rows are turned into float32 in shared memory once; warp w takes row w % RB and every (16 / RB)-th piece of
// 128 columns, 16 bytes a lane, for all NT tokens; the slices' sums are added in a fixed order.  z is [tokens, experts + 1].
template <typename T, int NT, int RB>
__global__ void __launch_bounds__(ROUTE_WARPS * 32)
moe_logits_kernel(const T *__restrict__ h, int64_t h_stride, const float *__restrict__ w_router,
                  const float *__restrict__ b_router, const float *__restrict__ w_gate, float *__restrict__ z, int tokens,
                  int width, int experts) {
  constexpr int KS = ROUTE_WARPS / RB;
  extern __shared__ __align__(16) float smem[];       // x [NT][width], partial sums [NT][RB][KS]
  float *xs = smem;
  float *part = smem + NT * width;
  le::let_successor_start();
  le::wait_for_predecessor();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t0 = blockIdx.x * NT;
  const int nt = tokens - t0 < NT ? tokens - t0 : NT;
  const int ld = experts + 1;
  const int rows = experts + (w_gate != nullptr ? 1 : 0);
  if (width % 4 == 0 && h_stride % 4 == 0 && reinterpret_cast<uintptr_t>(h) % 16 == 0) {
    const int quads = width >> 2;
    for (int i = threadIdx.x; i < NT * quads; i += blockDim.x) {
      const int j = i / quads, c = (i - j * quads) << 2;
      float v[4] = {};
      if (j < nt) unpack4(*reinterpret_cast<const typename RoutePiece<T>::type *>(h + static_cast<int64_t>(t0 + j) * h_stride + c), v);
      *reinterpret_cast<float4 *>(xs + j * width + c) = make_float4(v[0], v[1], v[2], v[3]);
    }
  } else {
    for (int i = threadIdx.x; i < NT * width; i += blockDim.x) {
      const int j = i / width, c = i - j * width;
      xs[i] = j < nt ? le::to_f32(h[static_cast<int64_t>(t0 + j) * h_stride + c]) : 0.0f;
    }
  }
  __syncthreads();
  const int rb = warp % RB, slice = warp / RB;
  const int r = blockIdx.y * RB + rb;
  float acc[NT] = {};
  if (r < rows) {
    const float *w = r < experts ? w_router + static_cast<int64_t>(r) * width : w_gate;
    const bool pieces = width % 4 == 0 && reinterpret_cast<uintptr_t>(w) % 16 == 0;
    if (pieces) {
#pragma unroll 4
      for (int c = (slice * 32 + lane) * 4; c < width; c += KS * 128) {
        const float4 wv = *reinterpret_cast<const float4 *>(w + c);
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          const float4 xv = *reinterpret_cast<const float4 *>(xs + j * width + c);
          acc[j] = fmaf(xv.x, wv.x, fmaf(xv.y, wv.y, fmaf(xv.z, wv.z, fmaf(xv.w, wv.w, acc[j]))));
        }
      }
    } else {
      for (int c = slice * 32 + lane; c < width; c += KS * 32) {
        const float wv = w[c];
#pragma unroll
        for (int j = 0; j < NT; ++j) acc[j] = fmaf(xs[j * width + c], wv, acc[j]);
      }
    }
  }
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    const float v = le::warp_sum(acc[j]);
    if (lane == 0) part[(j * RB + rb) * KS + slice] = v;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < NT * RB; i += blockDim.x) {
    const int j = i / RB, b = i - j * RB, row = blockIdx.y * RB + b;
    if (j >= nt || row >= rows) continue;
    float v = 0.0f;
    for (int k = 0; k < KS; ++k) v += part[(j * RB + b) * KS + k];
    if (row < experts && b_router != nullptr) v += b_router[row];
    z[static_cast<int64_t>(t0 + j) * ld + row] = v;
  }
}

// The choice: a warp per token picks the `top` largest of its logits (ties: the lower index), writes their ids and
// the softmax over them (`scoring` 0) or each one's own sigmoid (`scoring` 1), and the shared gate's sigmoid.  It
// marks what it has picked in z.
__global__ void moe_pick_kernel(float *__restrict__ z, int32_t *__restrict__ ids, float *__restrict__ weights,
                                float *__restrict__ gate, int tokens, int experts, int top, int with_gate, int scoring) {
  le::let_successor_start();
  le::wait_for_predecessor();
  const int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (t >= tokens) return;
  float *zt = z + static_cast<int64_t>(t) * (experts + 1);
  if (with_gate && lane == 0) gate[t] = 1.0f / (1.0f + expf(-zt[experts]));
  float first = 0.0f, total = 0.0f;
  for (int j = 0; j < top; ++j) {
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int e = lane; e < experts; e += 32) {
      const float v = zt[e];
      if (v > best || (v == best && e < at)) { best = v; at = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (ov > best || (ov == best && oa < at)) { best = ov; at = oa; }
    }
    if (at == 0x7fffffff) at = 0;   // (no finite logit left: cannot happen with top <= experts)
    if (j == 0) first = best;
    // scoring 1: the weight is the chosen logit's sigmoid by itself (the largest logits are the largest scores)
    const float p = scoring == 1 ? 1.0f / (1.0f + expf(-best)) : expf(best - first);
    total += p;
    if (lane == 0) {
      ids[static_cast<int64_t>(t) * top + j] = at;
      weights[static_cast<int64_t>(t) * top + j] = p;
      zt[at] = -INFINITY;
    }
    __syncwarp();
  }
  if (scoring == 1) return;
  for (int j = lane; j < top; j += 32) weights[static_cast<int64_t>(t) * top + j] /= total;
}

template <typename T, int NT, int RB>
int launch_logits(const void *h, int64_t h_stride, const float *w_router, const float *b_router, const float *w_gate, float *z,
                  int tokens, int width, int experts, cudaStream_t stream) {
  auto kernel = moe_logits_kernel<T, NT, RB>;
  const size_t smem = sizeof(float) * (static_cast<size_t>(NT) * width + NT * ROUTE_WARPS);
  if (smem > 48 * 1024) {
    static size_t raised = 0;            // per form and process: the most asked for so far
    if (smem > raised) {
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
      if (e != cudaSuccess) return le::invalid("le_moe_route: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
      raised = smem;
    }
  }
  const int rows = experts + (w_gate != nullptr ? 1 : 0);
  return le::launch_chained(kernel, dim3((tokens + NT - 1) / NT, (rows + RB - 1) / RB), dim3(ROUTE_WARPS * 32), smem, stream,
                            static_cast<const T *>(h), h_stride, w_router, b_router, w_gate, z, tokens, width, experts);
}

// One block.  meta[0] = number of tiles.  `padded`: every expert's slots start at a multiple of tile_m (slots that
// stand for no pair hold -1), so that a row tile of a product over the sorted rows lies within one expert; slots_cap
// is what slot_pair holds then.  pair_slot (or nullptr) receives each pair's slot.
__global__ void moe_group_kernel(const int32_t *__restrict__ ids, int pairs, int experts, int tile_m, int padded,
                                 int max_tiles, int slots_cap, int32_t *__restrict__ slot_pair,
                                 int32_t *__restrict__ pair_slot, int32_t *__restrict__ tile_expert,
                                 int32_t *__restrict__ tile_first, int32_t *__restrict__ tile_rows,
                                 int32_t *__restrict__ meta) {
  extern __shared__ int32_t ism[];
  int32_t *count = ism;                 // [experts]
  int32_t *offset = ism + experts;      // [experts + 1]
  int32_t *tile_at = offset + experts + 1;  // [experts + 1]
  le::let_successor_start();
  le::wait_for_predecessor();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) count[e] = 0;
  for (int k = threadIdx.x; k < max_tiles; k += blockDim.x) {
    tile_expert[k] = 0;
    tile_rows[k] = 0;
  }
  if (padded)
    for (int i = threadIdx.x; i < slots_cap; i += blockDim.x) slot_pair[i] = -1;
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int e = ids[p];
    if (e >= 0 && e < experts) atomicAdd(&count[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0, tiles = 0;
    for (int e = 0; e < experts; ++e) {
      offset[e] = padded ? tiles * tile_m : acc;
      tile_at[e] = tiles;
      acc += count[e];
      tiles += (count[e] + tile_m - 1) / tile_m;
    }
    offset[experts] = padded ? tiles * tile_m : acc;
    tile_at[experts] = tiles;
    meta[0] = tiles;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) {
    const int n = count[e];
    for (int i = 0, k = tile_at[e]; i < n; i += tile_m, ++k) {
      tile_expert[k] = e;
      tile_first[k] = offset[e] + i;
      tile_rows[k] = n - i < tile_m ? n - i : tile_m;
    }
    count[e] = 0;       // reused as the fill pointer
  }
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int e = ids[p];
    if (e >= 0 && e < experts) {
      const int slot = offset[e] + atomicAdd(&count[e], 1);
      slot_pair[slot] = p;
      if (pair_slot != nullptr) pair_slot[p] = slot;
    }
  }
}

// Rows of x gathered into slot order (16-byte pieces): out[slot] = x[slot_pair[slot] / src_div] (times the pair's
// weight where `pair_weight` is given), zeros for slots that stand for no pair; only the first meta[0] * tile_m
// slots are touched.
template <typename T>
__global__ void moe_gather_kernel(T *__restrict__ out, const T *__restrict__ x, int64_t x_stride,
                                  const int32_t *__restrict__ slot_pair, int src_div, int tile_m,
                                  const int32_t *__restrict__ meta, int width, const float *__restrict__ pair_weight) {
  le::let_successor_start();
  le::wait_for_predecessor();
  const int slot = blockIdx.x;
  if (slot >= meta[0] * tile_m) return;
  const int pair = slot_pair[slot];
  constexpr int PIECE = 16 / sizeof(T);
  uint4 *dst = reinterpret_cast<uint4 *>(out + static_cast<int64_t>(slot) * width);
  const uint4 *src = pair >= 0 ? reinterpret_cast<const uint4 *>(x + static_cast<int64_t>(pair / src_div) * x_stride) : nullptr;
  if (pair_weight != nullptr && src != nullptr) {      // the row times the pair's weight, rounded once
    const float f = pair_weight[pair];
    for (int i = threadIdx.x; i < width / PIECE; i += blockDim.x) {
      uint4 raw = src[i];
      T *e = reinterpret_cast<T *>(&raw);
#pragma unroll
      for (int v = 0; v < PIECE; ++v) e[v] = le::from_f32<T>(le::to_f32(e[v]) * f);
      dst[i] = raw;
    }
    return;
  }
  for (int i = threadIdx.x; i < width / PIECE; i += blockDim.x) dst[i] = src != nullptr ? src[i] : make_uint4(0, 0, 0, 0);
}

// out[t] = sum_j share[t, j] * y[pair_slot[t * top + j]] (+ gate[t] * shared[t]): the weighted sum over rows that
// lie in slot order.
template <typename T, typename TY>
__global__ void moe_combine_sorted_kernel(T *__restrict__ out, const TY *__restrict__ y, const int32_t *__restrict__ pair_slot,
                                          const float *__restrict__ share, const T *__restrict__ shared_out,
                                          const float *__restrict__ gate, int64_t n, int width, int top) {
  le::let_successor_start();
  le::wait_for_predecessor();
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int64_t t = i / width, c = i - t * width;
  float acc = 0.0f;
  for (int j = 0; j < top; ++j)
    acc = fmaf(share != nullptr ? share[t * top + j] : 1.0f,
               le::to_f32(y[static_cast<int64_t>(pair_slot[t * top + j]) * width + c]), acc);
  if (shared_out != nullptr) acc = fmaf(gate != nullptr ? gate[t] : 1.0f, le::to_f32(shared_out[i]), acc);
  out[i] = le::from_f32<T>(acc);
}

template <typename T, typename TOut, bool GATED>
__global__ void moe_grouped_kernel(TOut *__restrict__ out, int64_t out_stride, const T *__restrict__ a, int64_t a_stride,
                                   const T *__restrict__ w, int64_t expert_stride, int64_t w_stride,
                                   const int32_t *__restrict__ slot_pair, int src_div, int scatter,
                                   const float *__restrict__ pair_weight, const int32_t *__restrict__ tile_expert,
                                   const int32_t *__restrict__ tile_first, const int32_t *__restrict__ tile_rows,
                                   const int32_t *__restrict__ meta, int N, int K, le::GatedActivation act) {
  __shared__ float a_s[TILE_K][TILE_M + 1];
  __shared__ float w_s[GATED ? 2 : 1][TILE_K][TILE_N + 1];
  __shared__ int32_t src_row[TILE_M], dst_row[TILE_M];
  __shared__ float row_factor[TILE_M];
  le::let_successor_start();
  le::wait_for_predecessor();
  const int tile = blockIdx.y;
  if (tile >= meta[0]) return;
  const int expert = tile_expert[tile], first = tile_first[tile], rows = tile_rows[tile];
  const int n0 = blockIdx.x * TILE_N;
  if (threadIdx.x < TILE_M) {
    const int i = threadIdx.x;
    int src = 0, dst = 0;
    float f = 1.0f;
    if (i < rows) {
      const int pair = slot_pair[first + i];
      src = src_div > 0 ? pair / src_div : first + i;
      dst = scatter ? pair : first + i;
      if (pair_weight != nullptr) f = pair_weight[pair];
    }
    src_row[i] = src;
    dst_row[i] = dst;
    row_factor[i] = f;
  }
  __syncthreads();
  const T *w_e = w + static_cast<int64_t>(expert) * expert_stride;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;       // 16 x 16 threads: 2 rows x 4 columns each
  float acc[2][4] = {}, acc_up[2][4] = {};
  for (int k0 = 0; k0 < K; k0 += TILE_K) {
    for (int i = threadIdx.x; i < TILE_M * TILE_K; i += blockDim.x) {
      const int m = i / TILE_K, k = i - m * TILE_K;
      a_s[k][m] = (m < rows && k0 + k < K) ? le::to_f32(a[static_cast<int64_t>(src_row[m]) * a_stride + k0 + k]) : 0.0f;
    }
    for (int i = threadIdx.x; i < TILE_N * TILE_K; i += blockDim.x) {
      const int n = i / TILE_K, k = i - n * TILE_K;
      const bool in = n0 + n < N && k0 + k < K;
      w_s[0][k][n] = in ? le::to_f32(w_e[static_cast<int64_t>(n0 + n) * w_stride + k0 + k]) : 0.0f;
      if constexpr (GATED) w_s[1][k][n] = in ? le::to_f32(w_e[static_cast<int64_t>(N + n0 + n) * w_stride + k0 + k]) : 0.0f;
    }
    __syncthreads();
#pragma unroll 8
    for (int k = 0; k < TILE_K; ++k) {
      const float a0 = a_s[k][ty * 2], a1 = a_s[k][ty * 2 + 1];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float b = w_s[0][k][tx * 4 + j];
        acc[0][j] = fmaf(a0, b, acc[0][j]);
        acc[1][j] = fmaf(a1, b, acc[1][j]);
        if constexpr (GATED) {
          const float bu = w_s[1][k][tx * 4 + j];
          acc_up[0][j] = fmaf(a0, bu, acc_up[0][j]);
          acc_up[1][j] = fmaf(a1, bu, acc_up[1][j]);
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int m = ty * 2 + i;
    if (m >= rows) continue;
    TOut *o = out + static_cast<int64_t>(dst_row[m]) * out_stride;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if constexpr (GATED) {
        // (the pair's weight is the factor on the expert's input: both products carry it into the activation)
        v = le::gated_activation(v * row_factor[m], acc_up[i][j] * row_factor[m], act);
        o[n] = le::from_f32<TOut>(v);
      } else {
        o[n] = le::from_f32<TOut>(v * row_factor[m]);
      }
    }
  }
}


// ---- the same products on the tensor cores (bfloat16 inputs, mma.sync m16n8k16, float32 sums) ----
// A block takes one row tile (TM sorted slots of one expert) and TN output columns (gated: the TN gate rows and the
// TN up rows of W that make them).  Slots are the 16-row operand, W's rows the 8-column one; a warp owns 32 slots x
// WN columns.  K runs in steps through a ring of cp.async stages; rows of A are gathered through the slot list, rows
// beyond the tile and columns beyond K are filled with zeros by the copy itself.  K must be a multiple of 8 and all
// rows 16-byte aligned.
__device__ __forceinline__ void cp_async_16(void *smem, const void *gmem, int src_bytes) {
  const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(gmem), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// Two shapes.  Narrow (TM = 32 slots x 32 columns, K in steps of 64, four stages): few rows per expert, the product
// is bound by streaming W, so blocks are many and each keeps three stages of W in flight.  Wide (128 x 64, steps of
// 32, two stages): many rows per expert, where the tcgen05 product is not taken.
// Few (shape 16: the same 32 slots, named by its columns): a handful of row tiles in all (one or two decoded tokens),
// where only many small blocks with long steps of K keep the memory system busy.
template <int TM> struct MmaShape;
template <> struct MmaShape<32> { static constexpr int ROWS = 32, TN = 32, TK = 64, STAGES = 4, THREADS = 128, WARPS_M = 1; };
template <> struct MmaShape<128> { static constexpr int ROWS = 128, TN = 64, TK = 32, STAGES = 2, THREADS = 256, WARPS_M = 4; };
template <> struct MmaShape<16> { static constexpr int ROWS = 32, TN = 16, TK = 128, STAGES = 4, THREADS = 64, WARPS_M = 1; };

template <int SHAPE, bool GATED>
constexpr size_t mma_smem_bytes() {
  using S = MmaShape<SHAPE>;
  return static_cast<size_t>(S::STAGES) * (S::ROWS + (GATED ? 2 : 1) * S::TN) * (S::TK + 8) * sizeof(__nv_bfloat16);
}

template <int SHAPE, typename TOut, bool GATED>
__global__ void __launch_bounds__(MmaShape<SHAPE>::THREADS)
moe_grouped_mma_kernel(TOut *__restrict__ out, int64_t out_stride, const __nv_bfloat16 *__restrict__ a, int64_t a_stride,
                       const __nv_bfloat16 *__restrict__ w, int64_t expert_stride, int64_t w_stride,
                       const int32_t *__restrict__ slot_pair, int src_div, int scatter, const float *__restrict__ pair_weight,
                       const int32_t *__restrict__ tile_expert, const int32_t *__restrict__ tile_first,
                       const int32_t *__restrict__ tile_rows, const int32_t *__restrict__ meta, int N, int K,
                       le::GatedActivation act) {
  using S = MmaShape<SHAPE>;
  constexpr int TM = S::ROWS, TN = S::TN, TK = S::TK, STAGES = S::STAGES, THREADS = S::THREADS, WARPS_M = S::WARPS_M;
  constexpr int LD = TK + 8;                        // bf16 elements per shared-memory row: fragment loads free of bank conflicts
  constexpr int PIECES = TK / 8;                    // 16-byte pieces of a row of a stage
  constexpr int WARPS_N = THREADS / 32 / WARPS_M;
  constexpr int WN = TN / WARPS_N;                  // columns a warp owns
  constexpr int NT = WN / 8;                        // its 8-column tiles
  constexpr int WPARTS = GATED ? 2 : 1;
  constexpr int W_ROWS = WPARTS * TN;
  extern __shared__ __align__(16) unsigned char mma_smem[];
  __nv_bfloat16 *a_s = reinterpret_cast<__nv_bfloat16 *>(mma_smem);            // [STAGES][TM][LD]
  __nv_bfloat16 *w_s = a_s + STAGES * TM * LD;                                 // [STAGES][W_ROWS][LD]
  __shared__ int32_t src_row[TM], dst_row[TM];
  __shared__ float row_factor[TM];
  le::let_successor_start();
  le::wait_for_predecessor();
  const int tile = blockIdx.y;
  if (tile >= meta[0]) return;
  const int expert = tile_expert[tile], first = tile_first[tile], rows = tile_rows[tile];
  const int n0 = blockIdx.x * TN;
  for (int i = threadIdx.x; i < TM; i += THREADS) {
    int src = 0, dst = 0;
    float f = 1.0f;
    if (i < rows) {
      const int pair = slot_pair[first + i];
      src = src_div > 0 ? pair / src_div : first + i;
      dst = scatter ? pair : first + i;
      if (pair_weight != nullptr) f = pair_weight[pair];
    }
    src_row[i] = src;
    dst_row[i] = dst;
    row_factor[i] = f;
  }
  __syncthreads();
  const __nv_bfloat16 *w_e = w + static_cast<int64_t>(expert) * expert_stride;

  auto load_stage = [&](int stage, int k0) {
    // rows of x: only those the tile has (the others' shared memory is never read into a stored result)
    for (int i = threadIdx.x; i < TM * PIECES; i += THREADS) {
      const int m = i / PIECES, piece = i - m * PIECES, k = k0 + piece * 8;
      if (m >= rows) continue;
      const bool in = k < K;
      cp_async_16(a_s + (stage * TM + m) * LD + piece * 8, in ? a + static_cast<int64_t>(src_row[m]) * a_stride + k : a, in ? 16 : 0);
    }
    for (int i = threadIdx.x; i < W_ROWS * PIECES; i += THREADS) {
      const int r = i / PIECES, piece = i - r * PIECES, k = k0 + piece * 8;
      const int part = r / TN, n = n0 + r - part * TN;
      const bool in = n < N && k < K;
      cp_async_16(w_s + (stage * W_ROWS + r) * LD + piece * 8,
                  in ? w_e + static_cast<int64_t>(part * N + n) * w_stride + k : w_e, in ? 16 : 0);
    }
  };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int wm = (warp % WARPS_M) * 32, wn = (warp / WARPS_M) * WN;
  float acc[WPARTS][2][NT][4] = {};
  const int steps = (K + TK - 1) / TK;
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < steps) load_stage(s, s * TK);
    cp_async_commit();
  }
  for (int s = 0; s < steps; ++s) {
    cp_async_wait<STAGES - 2>();           // step s has landed
    __syncthreads();                       // ... for everyone, and everyone is done with step s - 1
    if (s + STAGES - 1 < steps) load_stage((s + STAGES - 1) % STAGES, (s + STAGES - 1) * TK);
    cp_async_commit();
    const int st = s % STAGES;
#pragma unroll
    for (int kk = 0; kk < TK; kk += 16) {
      uint32_t af[2][4];
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        const __nv_bfloat16 *base = a_s + (st * TM + wm + mt * 16) * LD + kk;
        af[mt][0] = *reinterpret_cast<const uint32_t *>(base + (g)*LD + 2 * t4);
        af[mt][1] = *reinterpret_cast<const uint32_t *>(base + (g + 8) * LD + 2 * t4);
        af[mt][2] = *reinterpret_cast<const uint32_t *>(base + (g)*LD + 2 * t4 + 8);
        af[mt][3] = *reinterpret_cast<const uint32_t *>(base + (g + 8) * LD + 2 * t4 + 8);
      }
#pragma unroll
      for (int part = 0; part < WPARTS; ++part)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const __nv_bfloat16 *base = w_s + (st * W_ROWS + part * TN + wn + nt * 8 + g) * LD + kk;
          uint32_t bf[2];
          bf[0] = *reinterpret_cast<const uint32_t *>(base + 2 * t4);
          bf[1] = *reinterpret_cast<const uint32_t *>(base + 2 * t4 + 8);
          mma_bf16_16816(acc[part][0][nt], af[0], bf);
          mma_bf16_16816(acc[part][1][nt], af[1], bf);
        }
    }
  }
  cp_async_wait<0>();
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int m = wm + mt * 16 + g + half * 8;
      if (m >= rows) continue;
      TOut *o = out + static_cast<int64_t>(dst_row[m]) * out_stride;
      const float f = row_factor[m];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int n = n0 + wn + nt * 8 + 2 * t4 + j;
          if (n >= N) continue;
          float v = acc[0][mt][nt][half * 2 + j];
          if constexpr (GATED) {
            v = le::gated_activation(v * f, acc[1][mt][nt][half * 2 + j] * f, act);
            o[n] = le::from_f32<TOut>(v);
          } else {
            o[n] = le::from_f32<TOut>(v * f);
          }
        }
    }
}

template <int TM, typename TOut, bool GATED, typename... Args>
int launch_grouped_mma(int N, int max_tiles, cudaStream_t stream, Args... args) {
  auto kernel = moe_grouped_mma_kernel<TM, TOut, GATED>;
  constexpr size_t smem = mma_smem_bytes<TM, GATED>();
  if (smem > 48 * 1024) {
    static bool raised = false;          // once per form and process
    if (!raised) {
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
      if (e != cudaSuccess) return le::invalid("le_moe_grouped: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
      raised = true;
    }
  }
  const dim3 grid((N + MmaShape<TM>::TN - 1) / MmaShape<TM>::TN, max_tiles);
  return le::launch_chained(kernel, grid, dim3(MmaShape<TM>::THREADS), smem, stream, args...);
}

template <typename T>
__global__ void moe_combine_kernel(T *__restrict__ out, const float *__restrict__ y, const T *__restrict__ shared_out,
                                   const float *__restrict__ gate, int64_t n, int width, int top) {
  le::let_successor_start();
  le::wait_for_predecessor();
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int64_t t = i / width, c = i - t * width;
  float acc = 0.0f;
  for (int j = 0; j < top; ++j) acc += y[(t * top + j) * width + c];
  if (shared_out != nullptr) acc = fmaf(gate != nullptr ? gate[t] : 1.0f, le::to_f32(shared_out[i]), acc);
  out[i] = le::from_f32<T>(acc);
}

}  // namespace

LE_API int le_moe_tile_rows(int wide) { return wide ? TILE_M_WIDE : TILE_M; }

// `z`: float32 scratch [tokens, experts + 1] (the logits; the picked ones are overwritten).
LE_API int le_moe_route(const void *h, int64_t h_stride, int dtype, const float *w_router, const float *b_router,
                        const float *w_gate, float *z, int32_t *ids, float *weights, float *gate, int tokens, int width,
                        int experts, int top, int scoring, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (top < 1 || top > experts) return le::invalid("le_moe_route: %d of %d experts", top, experts);
  // tokens a block takes: up to 8, fewer where the step has fewer or a row is wide
  int nt = 8;
  while (nt > 1 && (nt / 2 >= tokens || nt * width > ROUTE_SMEM_FLOATS)) nt >>= 1;
  if (static_cast<size_t>(width) * 4 > 200 * 1024) return le::invalid("le_moe_route: rows of %d values do not fit", width);
  // rows of the router a block takes: all 16 of a round where the tokens alone make enough blocks, else one row a
  // block with its warps sharing out the columns
  const bool many = (tokens + nt - 1) / nt >= 32;
  int rc;
#define LE_LOGITS(T, NT)                                                                                                  \
  rc = many ? launch_logits<T, NT, 16>(h, h_stride, w_router, b_router, w_gate, z, tokens, width, experts, stream)        \
            : launch_logits<T, NT, 1>(h, h_stride, w_router, b_router, w_gate, z, tokens, width, experts, stream)
  if (dtype == LE_BF16) {
    if (nt == 8) { LE_LOGITS(__nv_bfloat16, 8); }
    else if (nt == 4) { LE_LOGITS(__nv_bfloat16, 4); }
    else if (nt == 2) { LE_LOGITS(__nv_bfloat16, 2); }
    else { LE_LOGITS(__nv_bfloat16, 1); }
  } else {
    if (nt == 8) { LE_LOGITS(float, 8); }
    else if (nt == 4) { LE_LOGITS(float, 4); }
    else if (nt == 2) { LE_LOGITS(float, 2); }
    else { LE_LOGITS(float, 1); }
  }
#undef LE_LOGITS
  if (rc != 0) return rc;
  if (scoring != 0 && scoring != 1) return le::invalid("le_moe_route: scoring %d is neither 0 (softmax over the chosen) nor 1 (sigmoid)", scoring);
  return le::launch_chained(moe_pick_kernel, dim3((tokens + 7) / 8), dim3(256), 0, stream, z, ids, weights, gate, tokens, experts,
                            top, w_gate != nullptr ? 1 : 0, scoring);
}

LE_API int le_moe_group(const int32_t *ids, int pairs, int experts, int tile_m, int padded, int max_tiles, int slots_cap,
                        int32_t *slot_pair, int32_t *pair_slot, int32_t *tile_expert, int32_t *tile_first, int32_t *tile_rows,
                        int32_t *meta, cudaStream_t stream) {
  if (pairs <= 0) return 0;
  if (tile_m != TILE_M && tile_m != TILE_M_WIDE) return le::invalid("le_moe_group: row tiles of %d or %d, got %d", TILE_M, TILE_M_WIDE, tile_m);
  if (padded && slots_cap < max_tiles * tile_m) return le::invalid("le_moe_group: %d slots do not hold %d tiles of %d", slots_cap, max_tiles, tile_m);
  const size_t smem = sizeof(int32_t) * (3 * experts + 2);
  if (smem > 48 * 1024) return le::invalid("le_moe_group: too many experts (%d)", experts);
  return le::launch_chained(moe_group_kernel, dim3(1), dim3(1024), smem, stream, ids, pairs, experts, tile_m, padded, max_tiles,
                            slots_cap, slot_pair, pair_slot, tile_expert, tile_first, tile_rows, meta);
}

LE_API int le_moe_gather(void *out, const void *x, int64_t x_stride, int dtype, const int32_t *slot_pair, int src_div,
                         int tile_m, const int32_t *meta, int slots_cap, int width, const float *pair_weight,
                         cudaStream_t stream) {
  if (slots_cap <= 0) return 0;
  const int piece = dtype == LE_BF16 ? 8 : 4;
  if (width % piece || x_stride % piece || reinterpret_cast<uintptr_t>(out) % 16 || reinterpret_cast<uintptr_t>(x) % 16)
    return le::invalid("le_moe_gather: rows in 16-byte pieces only");
  if (dtype == LE_BF16)
    return le::launch_chained(moe_gather_kernel<__nv_bfloat16>, dim3(slots_cap), dim3(128), 0, stream,
                              static_cast<__nv_bfloat16 *>(out), static_cast<const __nv_bfloat16 *>(x), x_stride, slot_pair,
                              src_div, tile_m, meta, width, pair_weight);
  return le::launch_chained(moe_gather_kernel<float>, dim3(slots_cap), dim3(128), 0, stream, static_cast<float *>(out),
                            static_cast<const float *>(x), x_stride, slot_pair, src_div, tile_m, meta, width, pair_weight);
}

LE_API int le_moe_combine_sorted(void *out, int dtype, const void *y, int y_dtype, const int32_t *pair_slot,
                                 const float *share, const void *shared_out, const float *gate, int tokens, int width, int top,
                                 cudaStream_t stream) {
  const int64_t n = static_cast<int64_t>(tokens) * width;
  if (n <= 0) return 0;
  const dim3 grid(static_cast<unsigned>((n + 255) / 256)), block(256);
  if (dtype == LE_BF16 && y_dtype == LE_F32)
    return le::launch_chained(moe_combine_sorted_kernel<__nv_bfloat16, float>, grid, block, 0, stream,
                              static_cast<__nv_bfloat16 *>(out), static_cast<const float *>(y), pair_slot, share,
                              static_cast<const __nv_bfloat16 *>(shared_out), gate, n, width, top);
  if (dtype == LE_BF16 && y_dtype == LE_BF16)
    return le::launch_chained(moe_combine_sorted_kernel<__nv_bfloat16, __nv_bfloat16>, grid, block, 0, stream,
                              static_cast<__nv_bfloat16 *>(out), static_cast<const __nv_bfloat16 *>(y), pair_slot, share,
                              static_cast<const __nv_bfloat16 *>(shared_out), gate, n, width, top);
  if (dtype == LE_F32 && y_dtype == LE_F32)
    return le::launch_chained(moe_combine_sorted_kernel<float, float>, grid, block, 0, stream, static_cast<float *>(out),
                              static_cast<const float *>(y), pair_slot, share, static_cast<const float *>(shared_out), gate, n,
                              width, top);
  return le::invalid("le_moe_combine_sorted: no form for output type %d and rows of type %d", dtype, y_dtype);
}

// `max_tiles`: what the grid is sized for, pairs / tile_m + experts at most.  `tile_m`: the row tiles' size that
// le_moe_group was given: 32, or 128 (bfloat16 with 16-byte aligned rows only: the tensor-core form).
LE_API int le_moe_grouped(void *out, int out_dtype, int64_t out_stride, const void *a, int64_t a_stride, const void *w,
                          int64_t expert_stride, int64_t w_stride, int dtype, const int32_t *slot_pair, int src_div,
                          int scatter, const float *pair_weight, const int32_t *tile_expert, const int32_t *tile_first,
                          const int32_t *tile_rows, const int32_t *meta, int max_tiles, int tile_m, int N, int K, int gated,
                          int act_kind, float act_slope, float act_limit, cudaStream_t stream) {
  if (max_tiles <= 0 || N <= 0) return 0;
  if (max_tiles > 65535) return le::invalid("le_moe_grouped: %d row tiles are more than a grid holds", max_tiles);
  le::GatedActivation act;
  act.kind = act_kind;
  act.slope = act_slope;
  act.limit = act_limit;
  const bool aligned = K % 8 == 0 && a_stride % 8 == 0 && w_stride % 8 == 0 && expert_stride % 8 == 0 &&
                       reinterpret_cast<uintptr_t>(a) % 16 == 0 && reinterpret_cast<uintptr_t>(w) % 16 == 0;
  if (dtype == LE_BF16 && aligned && (tile_m == TILE_M || tile_m == TILE_M_WIDE)) {
#define LE_MOE_MMA(TM, TOut, GATED)                                                                                        \
  return launch_grouped_mma<TM, TOut, GATED>(N, max_tiles, stream, static_cast<TOut *>(out), out_stride,                   \
                                             static_cast<const __nv_bfloat16 *>(a), a_stride,                              \
                                             static_cast<const __nv_bfloat16 *>(w), expert_stride, w_stride, slot_pair,    \
                                             src_div, scatter, pair_weight, tile_expert, tile_first, tile_rows, meta, N, K, \
                                             act)
    if (tile_m == TILE_M && max_tiles <= 4) {
      if (gated && out_dtype == LE_BF16) LE_MOE_MMA(16, __nv_bfloat16, true);
      if (!gated && out_dtype == LE_F32) LE_MOE_MMA(16, float, false);
      if (!gated && out_dtype == LE_BF16) LE_MOE_MMA(16, __nv_bfloat16, false);
    } else if (tile_m == TILE_M) {
      if (gated && out_dtype == LE_BF16) LE_MOE_MMA(32, __nv_bfloat16, true);
      if (!gated && out_dtype == LE_F32) LE_MOE_MMA(32, float, false);
      if (!gated && out_dtype == LE_BF16) LE_MOE_MMA(32, __nv_bfloat16, false);
    } else {
      if (gated && out_dtype == LE_BF16) LE_MOE_MMA(128, __nv_bfloat16, true);
      if (!gated && out_dtype == LE_F32) LE_MOE_MMA(128, float, false);
      if (!gated && out_dtype == LE_BF16) LE_MOE_MMA(128, __nv_bfloat16, false);
    }
#undef LE_MOE_MMA
  }
  if (tile_m != TILE_M) return le::invalid("le_moe_grouped: the FP32-pipe form takes row tiles of %d, got %d", TILE_M, tile_m);
  const dim3 grid((N + TILE_N - 1) / TILE_N, max_tiles), block(256);
#define LE_MOE_LAUNCH(T, TOut, GATED)                                                                                         \
  return le::launch_chained(moe_grouped_kernel<T, TOut, GATED>, grid, block, 0, stream, static_cast<TOut *>(out), out_stride, \
                            static_cast<const T *>(a), a_stride, static_cast<const T *>(w), expert_stride, w_stride,          \
                            slot_pair, src_div, scatter, pair_weight, tile_expert, tile_first, tile_rows, meta, N, K, act)
  if (dtype == LE_BF16) {
    if (gated && out_dtype == LE_BF16) LE_MOE_LAUNCH(__nv_bfloat16, __nv_bfloat16, true);
    if (!gated && out_dtype == LE_F32) LE_MOE_LAUNCH(__nv_bfloat16, float, false);
    if (!gated && out_dtype == LE_BF16) LE_MOE_LAUNCH(__nv_bfloat16, __nv_bfloat16, false);
  } else if (out_dtype == LE_F32) {
    if (gated) LE_MOE_LAUNCH(float, float, true);
    LE_MOE_LAUNCH(float, float, false);
  }
#undef LE_MOE_LAUNCH
  return le::invalid("le_moe_grouped: no form for input type %d, output type %d, gated %d", dtype, out_dtype, gated);
}

LE_API int le_moe_combine(void *out, int dtype, const float *y, const void *shared_out, const float *gate, int tokens,
                          int width, int top, cudaStream_t stream) {
  const int64_t n = static_cast<int64_t>(tokens) * width;
  if (n <= 0) return 0;
  const dim3 grid(static_cast<unsigned>((n + 255) / 256)), block(256);
  if (dtype == LE_BF16)
    return le::launch_chained(moe_combine_kernel<__nv_bfloat16>, grid, block, 0, stream, static_cast<__nv_bfloat16 *>(out), y,
                              static_cast<const __nv_bfloat16 *>(shared_out), gate, n, width, top);
  return le::launch_chained(moe_combine_kernel<float>, grid, block, 0, stream, static_cast<float *>(out), y,
                            static_cast<const float *>(shared_out), gate, n, width, top);
}
