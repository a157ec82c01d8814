// Causal convolution over time on every channel, added to its own input, with
// the last inputs of each request kept as per-request state between steps:
//
//   out[t] = h[t] + sum_{j < taps} w[j] * h[t - (taps - 1 - j)]        (per channel)
//
// where h before the start of a request is zero.  A step brings any cut of a
// request's tokens (a whole prompt, a portion of two tokens, one decoded
// token); inputs from before the step come from the request's state row
// [taps - 1, channels], which holds the inputs at the taps - 1 positions before
// the step, oldest first, and is brought up to date here.
//
// Work is cut into tiles of 16 consecutive tokens of one request (the step's
// tile lists) times slices of channels; a thread owns one token of its tile and
// VEC neighbouring channels (one 16-byte access where the sizes allow it) and
// reads its token's earlier inputs from the step's rows, or, before the step's
// first token, from the state.  Only the block of a request's first tile
// touches that request's state for its channels: its threads read what they
// need of it, the block meets, and then the threads of the first taps - 1 rows
// write the new state, from the step's inputs (which this kernel only reads)
// and from old state they fetched before the meeting.  So one launch serves
// every cut.  Rows that stand for no request (slot < 0) see zeros before them
// and keep nothing.  In a step whose requests all bring one token
// (`tile_request` null) request b is tile b: no list is read.
//
// Sums are 32-bit, rounded once.
#include "common.cuh"

namespace {

constexpr int CONV_TILE = 16;       // tokens of a tile: one per group of CONV_LANES threads
constexpr int CONV_LANES = 8;       // threads side by side over channels
constexpr int CONV_THREADS = CONV_TILE * CONV_LANES;
constexpr int CONV_MAX_TAPS = CONV_TILE + 1;   // a tile must hold the taps - 1 inputs before the next tile

// VEC values at p as floats / from floats, in 16-byte accesses where VEC > 1 (p is then 16-byte aligned and VEC a
// multiple of the values one access holds).
template <typename T, int VEC>
__device__ __forceinline__ void load_channels(float (&dst)[VEC], const T *p) {
  if constexpr (VEC == 1) {
    dst[0] = le::to_f32(*p);
  } else {
    constexpr int PER = 16 / sizeof(T);
    static_assert(VEC % PER == 0, "whole 16-byte accesses");
#pragma unroll
    for (int i = 0; i < VEC; i += PER) {
      const uint4 raw = *reinterpret_cast<const uint4 *>(p + i);
      const T *e = reinterpret_cast<const T *>(&raw);
#pragma unroll
      for (int v = 0; v < PER; ++v) dst[i + v] = le::to_f32(e[v]);
    }
  }
}
template <typename T, int VEC>
__device__ __forceinline__ void store_channels(T *p, const float (&src)[VEC]) {
  if constexpr (VEC == 1) {
    *p = le::from_f32<T>(src[0]);
  } else {
    constexpr int PER = 16 / sizeof(T);
    static_assert(VEC % PER == 0, "whole 16-byte accesses");
#pragma unroll
    for (int i = 0; i < VEC; i += PER) {
      uint4 raw;
      T *e = reinterpret_cast<T *>(&raw);
#pragma unroll
      for (int v = 0; v < PER; ++v) e[v] = le::from_f32<T>(src[i + v]);
      *reinterpret_cast<uint4 *>(p + i) = raw;
    }
  }
}

template <typename T, int VEC>
__global__ void __launch_bounds__(CONV_THREADS)
short_conv_kernel(T *__restrict__ out, const T *__restrict__ h, const float *__restrict__ w, float *__restrict__ state,
                  int num_state_rows, const int32_t *__restrict__ state_slots, const int32_t *__restrict__ cu_q,
                  const int32_t *__restrict__ tile_request, const int32_t *__restrict__ tile_q0, int channels, int taps,
                  int64_t h_stride, int add_input, int activation, const float *__restrict__ bias) {
  le::let_successor_start();
  const int r = threadIdx.x / CONV_LANES;                                   // this thread's token within the tile
  const int c = (blockIdx.y * CONV_LANES + threadIdx.x % CONV_LANES) * VEC;  // its first channel
  const bool in_range = c < channels;
  const int keep = taps - 1;
  int b, q0, first, q_len;
  // (the step's integers do not depend on the kernel before this one)
  if (tile_request) {
    b = tile_request[blockIdx.x], q0 = tile_q0[blockIdx.x];
    first = cu_q[b], q_len = cu_q[b + 1] - first;
  } else {
    b = blockIdx.x, q0 = 0, first = b, q_len = 1;
  }
  const int q = q0 + r;                  // index of this token among the request's tokens in the step
  const bool live = in_range && q < q_len;
  float *mine = nullptr;
  if (q0 == 0 && keep > 0 && in_range) {
    const int slot = state_slots[b];
    if (slot >= 0 && slot < num_state_rows) mine = state + (static_cast<int64_t>(slot) * keep) * channels + c;
  }
  // what this thread will write into the state comes from the old state where the step is shorter than taps - 1:
  // fetched before the block meets (state row r becomes the input taps - 1 - r steps before the step's end)
  const int new_src = q_len - keep + r;
  const bool writes_state = mine != nullptr && r < keep;
  float carry[VEC];
#pragma unroll
  for (int e = 0; e < VEC; ++e) carry[e] = 0.0f;
  if (writes_state && new_src < 0) load_channels<float, VEC>(carry, mine + static_cast<int64_t>(keep + new_src) * channels);

  le::wait_for_predecessor();
  const T *hx = h + static_cast<int64_t>(first) * h_stride + c;
  if (live) {
    float acc[VEC];
    if (add_input) {
      load_channels<T, VEC>(acc, hx + static_cast<int64_t>(q) * h_stride);
    } else {
#pragma unroll
      for (int e = 0; e < VEC; ++e) acc[e] = 0.0f;
    }
    if (bias != nullptr) {       // one number per channel, the sum's first term
      float bv[VEC];
      load_channels<float, VEC>(bv, bias + c);
#pragma unroll
      for (int e = 0; e < VEC; ++e) acc[e] += bv[e];
    }
    for (int j = 0; j < taps; ++j) {
      const int src = q - (keep - j);
      float v[VEC], wt[VEC];
      load_channels<float, VEC>(wt, w + static_cast<int64_t>(j) * channels + c);
      if (src >= 0) {
        load_channels<T, VEC>(v, hx + static_cast<int64_t>(src) * h_stride);
      } else if (mine) {          // (src < 0 only in the request's first tile)
        load_channels<float, VEC>(v, mine + static_cast<int64_t>(keep + src) * channels);
      } else {
#pragma unroll
        for (int e = 0; e < VEC; ++e) v[e] = 0.0f;
      }
#pragma unroll
      for (int e = 0; e < VEC; ++e) acc[e] = fmaf(wt[e], v[e], acc[e]);
    }
    if (activation == 1) {
#pragma unroll
      for (int e = 0; e < VEC; ++e) acc[e] = acc[e] / (1.0f + expf(-acc[e]));
    }
    store_channels<T, VEC>(out + (static_cast<int64_t>(first) + q) * channels + c, acc);
  }
  __syncthreads();       // every read of the old state is done
  if (writes_state) {
    if (new_src >= 0) load_channels<T, VEC>(carry, hx + static_cast<int64_t>(new_src) * h_stride);
    store_channels<float, VEC>(mine + static_cast<int64_t>(r) * channels, carry);
  }
}

}  // namespace

// The general form: rows of h are h_stride elements apart (the channels are the first `channels` columns of wider
// rows); add_input 0 leaves the token's own input out of the sum (a plain convolution, whose last tap is the current
// token's); activation 1 puts silu over the sum; bias (float32 [channels] or null) is added to the sum.
LE_API int le_short_conv_general(void *out, const void *h, int64_t h_stride, int dtype, const float *w, float *state,
                                 int num_state_rows, const int32_t *state_slots, const int32_t *cu_q,
                                 const int32_t *tile_request, const int32_t *tile_q0, int num_tiles, int tile, int channels,
                                 int taps, int add_input, int activation, const float *bias, cudaStream_t stream);

// out, h: [tokens, channels] contiguous (different buffers); w: [taps, channels] float32; state:
// [num_state_rows, taps - 1, channels] float32 (may be null when taps is 1); the tiles list `tile` tokens each.
// tile_request and tile_q0 null: every request of the step brings one token, and there are `num_tiles` of them.
LE_API int le_short_conv(void *out, const void *h, int dtype, const float *w, float *state, int num_state_rows,
                         const int32_t *state_slots, const int32_t *cu_q, const int32_t *tile_request,
                         const int32_t *tile_q0, int num_tiles, int tile, int channels, int taps, cudaStream_t stream) {
  return le_short_conv_general(out, h, channels, dtype, w, state, num_state_rows, state_slots, cu_q, tile_request, tile_q0,
                               num_tiles, tile, channels, taps, 1, 0, nullptr, stream);
}

LE_API int le_short_conv_general(void *out, const void *h, int64_t h_stride, int dtype, const float *w, float *state,
                                 int num_state_rows, const int32_t *state_slots, const int32_t *cu_q,
                                 const int32_t *tile_request, const int32_t *tile_q0, int num_tiles, int tile, int channels,
                                 int taps, int add_input, int activation, const float *bias, cudaStream_t stream) {
  if (num_tiles <= 0 || channels <= 0) return 0;
  if (h_stride < channels) return le::invalid("le_short_conv: rows of %lld elements hold no %d channels", (long long)h_stride, channels);
  if (taps < 1 || taps > CONV_MAX_TAPS) return le::invalid("le_short_conv: taps must be 1..%d, got %d", CONV_MAX_TAPS, taps);
  if (tile != CONV_TILE) return le::invalid("le_short_conv: the tiles must list %d tokens each, not %d", CONV_TILE, tile);
  if (out == h) return le::invalid("le_short_conv: out and h must be different buffers");
  if ((tile_request == nullptr) != (tile_q0 == nullptr)) return le::invalid("le_short_conv: both tile lists or neither");
  const int vec = dtype == LE_BF16 ? 8 : 4;
  // 16-byte accesses to the rows (vec values of the type) and to weights and state (two or one of them per access)
  const bool wide = channels % 8 == 0 && h_stride % 8 == 0 &&
                    ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(h) | reinterpret_cast<uintptr_t>(w) |
                      reinterpret_cast<uintptr_t>(state) | reinterpret_cast<uintptr_t>(bias)) & 15) == 0;
  const int per_block = CONV_LANES * (wide ? vec : 1);
  const dim3 grid(num_tiles, (channels + per_block - 1) / per_block);
  if (grid.y > 65535) return le::invalid("le_short_conv: too many channels for one launch");
#define LE_GO(T, V)                                                                                                  \
  return le::launch_chained(short_conv_kernel<T, V>, grid, dim3(CONV_THREADS), 0, stream, static_cast<T *>(out),     \
                            static_cast<const T *>(h), w, state, num_state_rows, state_slots, cu_q, tile_request,    \
                            tile_q0, channels, taps, h_stride, add_input, activation, bias)
  if (dtype == LE_BF16) { if (wide) LE_GO(__nv_bfloat16, 8); LE_GO(__nv_bfloat16, 1); }
  if (dtype == LE_F32) { if (wide) LE_GO(float, 4); LE_GO(float, 1); }
#undef LE_GO
  return le::invalid("le_short_conv: unknown dtype code %d", dtype);
}
