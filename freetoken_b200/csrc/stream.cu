// Kernels around the 32-bit residual stream for layers that are not "add one tensor, RMS-norm the sum":
//
//   * stream_add_norm: adds up to five kinds of rows to the stream in one pass (two dense sub-layer
//     outputs, the sum over a token's expert routes, rows of a table picked by token id, one vector
//     for every token) and applies a norm that needs no statistics of the row (Dynamic Tanh,
//     y = tanh(alpha z) w + b), or none at all.  Every sum is taken in 32 bits and the stream is
//     stored in 32 bits.  A parallel layer (one norm feeding mixer and feed-forward, both outputs
//     added) and the re-injection of the input embedding before a repeated range of layers both
//     come down to this.
//   * head_gate: o[t, h, :] *= sigmoid(g[t, h]), the per-head output gate of an attention mixer.
//   * table_route: expert ids of a token read from a [vocab, top] table by its token id, equal weights.
//   * scale_f32: x *= s (logit scale).
#include "common.cuh"

namespace ftk {

struct StreamArgs {
  FtkStreamNorm a;
};

template <typename T>
__device__ __forceinline__ float stream_row_value(const FtkStreamNorm& a, int src_row, size_t src, int i, int tok) {
  float z = a.residual ? a.residual[src + i] : 0.f;
  if (a.x1) z += to_float(((const T*)a.x1)[src + i]);
  if (a.x2) z += to_float(((const T*)a.x2)[src + i]);
  if (a.y) {
    float acc = 0.f;
    for (int j = 0; j < a.top_k; ++j) {  // route order
      const int p = a.route_pos[(size_t)src_row * a.top_k + j];
      if (p >= 0 && p < a.n_routes) acc += to_float(((const T*)a.y)[(size_t)p * a.hidden + i]);
    }
    z += acc;
  }
  if (a.table && tok >= 0) z += to_float(((const T*)a.table)[(size_t)tok * a.hidden + i]);
  if (a.vec) z += a.vec[i];
  return z;
}

template <typename T>
__global__ void stream_add_norm_kernel(StreamArgs args) {
  pdl_wait();
  pdl_trigger();
  const FtkStreamNorm& a = args.a;
  const int r = blockIdx.x;
  const int src_row = a.rows ? a.rows[r] : r;
  const size_t src = (size_t)src_row * a.hidden, dst = (size_t)r * a.hidden;
  const bool update = a.rows == nullptr && a.residual != nullptr && (a.x1 || a.x2 || a.y || a.table || a.vec);
  int tok = -1;
  if (a.table) {
    tok = a.ids[src_row];
    if (tok < 0 || tok >= a.vocab) tok = -1;  // an id outside the table adds nothing, never a fault
  }
  const float alpha = a.norm == 1 ? a.alpha[0] : 0.f;
  for (int i = threadIdx.x; i < a.hidden; i += blockDim.x) {
    const float z = stream_row_value<T>(a, src_row, src, i, tok);
    if (update) a.residual[src + i] = z;
    if (a.out) {
      const float y = a.norm == 1 ? tanhf(alpha * z) * a.weight[i] + a.bias[i] : z;
      ((T*)a.out)[dst + i] = from_float<T>(y);
    }
  }
}

// The same, four consecutive elements per thread (rows of a multiple of 8 elements, 16-byte aligned tensors).
template <typename T>
__device__ __forceinline__ void load4(const T* p, float (&v)[4]);
template <>
__device__ __forceinline__ void load4<float>(const float* p, float (&v)[4]) {
  const float4 t = *reinterpret_cast<const float4*>(p);
  v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
template <>
__device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[4]) {
  const uint2 t = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&t.x);
  const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&t.y);
  v[0] = __low2float(lo); v[1] = __high2float(lo); v[2] = __low2float(hi); v[3] = __high2float(hi);
}
template <typename T>
__device__ __forceinline__ void store4(T* p, const float (&v)[4]);
template <>
__device__ __forceinline__ void store4<float>(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
template <>
__device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[4]) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]);
  const __nv_bfloat162 hi = __floats2bfloat162_rn(v[2], v[3]);
  uint2 t;
  t.x = *reinterpret_cast<const uint32_t*>(&lo);
  t.y = *reinterpret_cast<const uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = t;
}

template <typename T>
__global__ void stream_add_norm_vec_kernel(StreamArgs args) {
  pdl_wait();
  pdl_trigger();
  const FtkStreamNorm& a = args.a;
  const int r = blockIdx.x;
  const int src_row = a.rows ? a.rows[r] : r;
  const size_t src = (size_t)src_row * a.hidden, dst = (size_t)r * a.hidden;
  const bool update = a.rows == nullptr && a.residual != nullptr && (a.x1 || a.x2 || a.y || a.table || a.vec);
  int tok = -1;
  if (a.table) {
    tok = a.ids[src_row];
    if (tok < 0 || tok >= a.vocab) tok = -1;
  }
  const float alpha = a.norm == 1 ? a.alpha[0] : 0.f;
  for (int i = threadIdx.x * 4; i < a.hidden; i += blockDim.x * 4) {
    float z[4] = {0.f, 0.f, 0.f, 0.f}, t[4];
    if (a.residual) load4<float>(a.residual + src + i, z);
    if (a.x1) {
      load4<T>((const T*)a.x1 + src + i, t);
#pragma unroll
      for (int q = 0; q < 4; ++q) z[q] += t[q];
    }
    if (a.x2) {
      load4<T>((const T*)a.x2 + src + i, t);
#pragma unroll
      for (int q = 0; q < 4; ++q) z[q] += t[q];
    }
    if (a.y) {
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      for (int j = 0; j < a.top_k; ++j) {
        const int p = __ldg(a.route_pos + (size_t)src_row * a.top_k + j);
        if (p >= 0 && p < a.n_routes) {
          load4<T>((const T*)a.y + (size_t)p * a.hidden + i, t);
#pragma unroll
          for (int q = 0; q < 4; ++q) acc[q] += t[q];
        }
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) z[q] += acc[q];
    }
    if (a.table && tok >= 0) {
      load4<T>((const T*)a.table + (size_t)tok * a.hidden + i, t);
#pragma unroll
      for (int q = 0; q < 4; ++q) z[q] += t[q];
    }
    if (a.vec) {
      load4<float>(a.vec + i, t);
#pragma unroll
      for (int q = 0; q < 4; ++q) z[q] += t[q];
    }
    if (update) store4<float>(a.residual + src + i, z);
    if (a.out) {
      if (a.norm == 1) {
        float w[4], b[4];
        load4<float>(a.weight + i, w);
        load4<float>(a.bias + i, b);
#pragma unroll
        for (int q = 0; q < 4; ++q) z[q] = tanhf(alpha * z[q]) * w[q] + b[q];
      }
      store4<T>((T*)a.out + dst + i, z);
    }
  }
}

// o[t, h, :] *= sigmoid(g[t * g_stride + h]); one warp per (token, head)
template <typename T>
__global__ void head_gate_kernel(T* __restrict__ o, const T* __restrict__ g, long long g_stride, int n_tokens,
                                 int n_heads, int head_dim) {
  pdl_wait();
  pdl_trigger();
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= (long long)n_tokens * n_heads) return;
  const int lane = threadIdx.x & 31;
  const long long t = w / n_heads;
  const int h = (int)(w % n_heads);
  const float x = to_float(g[t * g_stride + h]);
  const float s = 1.f / (1.f + expf(-x));
  T* row = o + (size_t)w * head_dim;
  for (int d = lane; d < head_dim; d += 32) row[d] = from_float<T>(to_float(row[d]) * s);
}

__global__ void table_route_kernel(const int32_t* __restrict__ token_ids, const int32_t* __restrict__ table, int n_tokens,
                                   int vocab, int top_k, int n_experts, float weight, int32_t* __restrict__ ids,
                                   float* __restrict__ weights) {
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_tokens * top_k) return;
  const int t = i / top_k, j = i % top_k;
  int tok = token_ids[t];
  tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
  int e = table[(size_t)tok * top_k + j];
  e = e < 0 ? 0 : (e >= n_experts ? n_experts - 1 : e);  // a bad table entry names some expert, never memory outside the banks
  ids[i] = e;
  weights[i] = weight;
}

__global__ void scale_f32_kernel(float* x, long long n, float s) {
  pdl_wait();
  pdl_trigger();
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (; i < n; i += stride) x[i] *= s;
}

static inline bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace ftk

using namespace ftk;

extern "C" int ftk_stream_add_norm(const FtkStreamNorm* a, void* stream) {
  FTK_REQUIRE(a != nullptr, "stream_add_norm: null arguments");
  FTK_REQUIRE(dtype_ok(a->dtype), "stream_add_norm: bad dtype %d", a->dtype);
  FTK_REQUIRE(a->n_rows >= 0 && a->hidden > 0, "stream_add_norm: bad sizes rows=%d H=%d", a->n_rows, a->hidden);
  if (a->n_rows == 0) return 0;
  FTK_REQUIRE(a->residual || a->x1 || a->x2 || a->y || a->table, "stream_add_norm: nothing to add up");
  FTK_REQUIRE(a->residual || a->out, "stream_add_norm: nowhere to write");
  FTK_REQUIRE(!a->y || (a->route_pos && a->top_k >= 1 && a->n_routes >= 0), "stream_add_norm: routed rows need their positions");
  FTK_REQUIRE(!a->table || (a->ids && a->vocab >= 1), "stream_add_norm: table rows need token ids");
  FTK_REQUIRE(a->norm == 0 || a->norm == 1, "stream_add_norm: unknown norm %d", a->norm);
  FTK_REQUIRE(a->norm == 0 || (a->weight && a->bias && a->alpha && a->out), "stream_add_norm: the norm needs weight, bias, alpha and out");
  StreamArgs args;
  args.a = *a;
  cudaStream_t s = (cudaStream_t)stream;
  const bool vec = a->hidden % 8 == 0 && al16(a->residual) && al16(a->x1) && al16(a->x2) && al16(a->y) && al16(a->table) &&
                   al16(a->vec) && al16(a->weight) && al16(a->bias) && al16(a->out);
  if (vec) {
    int threads = (a->hidden / 4 + 31) / 32 * 32;
    threads = threads > 256 ? 256 : threads;
    if (a->dtype == FTK_F32) FTK_LAUNCH(stream_add_norm_vec_kernel<float>, a->n_rows, threads, 0, s, args);
    else FTK_LAUNCH(stream_add_norm_vec_kernel<__nv_bfloat16>, a->n_rows, threads, 0, s, args);
  } else {
    int threads = (a->hidden + 31) / 32 * 32;
    threads = threads > 256 ? 256 : threads;
    if (a->dtype == FTK_F32) FTK_LAUNCH(stream_add_norm_kernel<float>, a->n_rows, threads, 0, s, args);
    else FTK_LAUNCH(stream_add_norm_kernel<__nv_bfloat16>, a->n_rows, threads, 0, s, args);
  }
  FTK_LAUNCH_CHECK("stream_add_norm");
  return 0;
}

extern "C" int ftk_head_gate(void* o, int dtype, const void* gates, long long gate_stride, int n_tokens, int n_heads,
                             int head_dim, void* stream) {
  FTK_REQUIRE(dtype_ok(dtype), "head_gate: bad dtype %d", dtype);
  FTK_REQUIRE(n_tokens >= 0 && n_heads >= 1 && head_dim >= 1 && gate_stride >= n_heads, "head_gate: bad sizes");
  if (n_tokens == 0) return 0;
  FTK_REQUIRE(o && gates, "head_gate: null pointer");
  const long long warps = (long long)n_tokens * n_heads;
  const long long blocks = (warps + 3) / 4;
  FTK_REQUIRE(blocks <= 0x7fffffffLL, "head_gate: too many rows");
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == FTK_F32)
    FTK_LAUNCH(head_gate_kernel<float>, (int)blocks, 128, 0, s, (float*)o, (const float*)gates, gate_stride, n_tokens, n_heads, head_dim);
  else
    FTK_LAUNCH(head_gate_kernel<__nv_bfloat16>, (int)blocks, 128, 0, s, (__nv_bfloat16*)o, (const __nv_bfloat16*)gates, gate_stride,
               n_tokens, n_heads, head_dim);
  FTK_LAUNCH_CHECK("head_gate");
  return 0;
}

extern "C" int ftk_table_route(const int32_t* token_ids, const int32_t* table, int n_tokens, int vocab, int top_k,
                               int n_experts, float weight, int32_t* ids, float* weights, void* stream) {
  FTK_REQUIRE(n_tokens >= 0 && vocab >= 1 && top_k >= 1 && n_experts >= 1, "table_route: bad sizes");
  if (n_tokens == 0) return 0;
  FTK_REQUIRE(token_ids && table && ids && weights, "table_route: null pointer");
  const long long n = (long long)n_tokens * top_k;
  FTK_REQUIRE(n <= 0x7fffffffLL, "table_route: too many routes");
  // (an ordinary launch order: the kernels after it read the ids before their own wait on the kernel before)
  FTK_LAUNCH(table_route_kernel, (int)((n + 127) / 128), 128, 0, (cudaStream_t)stream, token_ids, table, n_tokens, vocab, top_k,
             n_experts, weight, ids, weights);
  FTK_LAUNCH_CHECK("table_route");
  return 0;
}

extern "C" int ftk_scale_f32(float* x, long long n, float s, void* stream) {
  FTK_REQUIRE(n >= 0 && (n == 0 || x), "scale_f32: bad arguments");
  if (n == 0) return 0;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  FTK_LAUNCH(scale_f32_kernel, (int)blocks, 256, 0, (cudaStream_t)stream, x, n, s);
  FTK_LAUNCH_CHECK("scale_f32");
  return 0;
}
