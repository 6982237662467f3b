// Kernels of layers that norm a sub-layer on both sides, of gated head outputs and of capped logits.
//
//   * postnorm_add_norm: a sub-layer's output a is normed before it joins the 32-bit stream, and the
//     stream is normed for the next sub-layer in the same pass:
//         r <- r + a * rsqrt(mean(a^2) + eps_a) * w_a ;  out = r * rsqrt(mean(r^2) + eps_r) * w_r
//     (w = 1 + weight in the Gemma form).  a is a dense row, or the sum over a token's expert routes
//     (+ the shared expert's row), taken in 32 bits in route order.  Either half can be left out: without
//     w_r only the stream is updated, with `rows` only those rows are normed and the stream stays.
//   * gated_heads: per (token, head) row, an optional RMS norm over the head (plain weight) and a gate taken
//     element by element from another projection of the same token: y = norm(x) * act(g), act = sigmoid or
//     silu.  The input is 32-bit (a recurrent layer's output) or the engine's type (attention output, in place).
//   * softcap: x <- cap * tanh(x / cap) on float32 logits.
#include "common.cuh"

namespace ftk {

struct SandwichArgs {
  const void* x;          // [*, hidden] dense rows of the sub-layer's output, or the experts' rows when route_pos is set
  const int32_t* route_pos;
  int top_k, n_routes;
  const void* shared;     // [*, hidden] or null (with route_pos)
  const float* post_w;    // [hidden]
  float* residual;        // [*, hidden]
  const float* pre_w;     // [hidden] or null: no norm of the stream, no out
  void* out;              // [n_rows, hidden] of the engine's type, or null
  float* out_f32;         // [n_rows, hidden] or null
  const int32_t* rows;    // or null
  int n_rows, hidden;
  float post_eps, pre_eps;
  int post_gemma, pre_gemma;
};

// One block per row.  Everything the row needs from memory (the sub-layer's output, the stream, both weights) is
// asked for in the first pass, four elements a thread at a time where the row allows it; the second and third
// pass work from shared memory and registers.  `arow` holds a * w_a, `zrow` the stream's row, then the sum.
template <typename T, bool VEC>
__global__ void __launch_bounds__(256) postnorm_add_norm_kernel(SandwichArgs a) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ __align__(16) float srow[];
  __shared__ float red[33];
  float* arow = srow;
  float* zrow = srow + a.hidden;
  const int r = blockIdx.x;
  const int src_row = a.rows ? a.rows[r] : r;
  const size_t src = (size_t)src_row * a.hidden, dst = (size_t)r * a.hidden;
  const T* x = (const T*)a.x;
  const T* shared = (const T*)a.shared;
  constexpr int W = VEC ? 4 : 1;
  float ss = 0.f;
  for (int i = threadIdx.x * W; i < a.hidden; i += blockDim.x * W) {
    float v[4], res[4], wa[4];
    if constexpr (VEC) {
      Vec4<float>::load(a.residual + src + i, res);
      Vec4<float>::load(a.post_w + i, wa);
    } else {
      res[0] = a.residual[src + i];
      wa[0] = a.post_w[i];
    }
    if (a.route_pos) {
#pragma unroll
      for (int u = 0; u < W; ++u) v[u] = 0.f;
      for (int j = 0; j < a.top_k; ++j) {  // route order
        const int p = a.route_pos[(size_t)src_row * a.top_k + j];
        if (p >= 0 && p < a.n_routes) {
          float y[4];
          if constexpr (VEC) Vec4<T>::load(x + (size_t)p * a.hidden + i, y);
          else y[0] = to_float(x[(size_t)p * a.hidden + i]);
#pragma unroll
          for (int u = 0; u < W; ++u) v[u] += y[u];
        }
      }
      if (shared) {
        float y[4];
        if constexpr (VEC) Vec4<T>::load(shared + src + i, y);
        else y[0] = to_float(shared[src + i]);
#pragma unroll
        for (int u = 0; u < W; ++u) v[u] += y[u];
      }
    } else {
      if constexpr (VEC) Vec4<T>::load(x + src + i, v);
      else v[0] = to_float(x[src + i]);
    }
#pragma unroll
    for (int u = 0; u < W; ++u) {
      ss += v[u] * v[u];
      arow[i + u] = v[u] * (a.post_gemma ? 1.f + wa[u] : wa[u]);
      zrow[i + u] = res[u];
    }
  }
  ss = block_sum(ss, red);
  const float inv_a = rsqrtf(ss / (float)a.hidden + a.post_eps);
  float ss2 = 0.f;
  for (int i = threadIdx.x * W; i < a.hidden; i += blockDim.x * W) {
    float z[4];
#pragma unroll
    for (int u = 0; u < W; ++u) {
      z[u] = zrow[i + u] + arow[i + u] * inv_a;
      zrow[i + u] = z[u];
      ss2 += z[u] * z[u];
    }
    if (!a.rows) {
      if constexpr (VEC) Vec4<float>::store(a.residual + src + i, z);
      else a.residual[src + i] = z[0];
    }
  }
  if (!a.pre_w) return;
  ss2 = block_sum(ss2, red);
  const float inv_r = rsqrtf(ss2 / (float)a.hidden + a.pre_eps);
  T* out = (T*)a.out;
  for (int i = threadIdx.x * W; i < a.hidden; i += blockDim.x * W) {
    float wr[4], y[4];
    if constexpr (VEC) Vec4<float>::load(a.pre_w + i, wr);
    else wr[0] = a.pre_w[i];
#pragma unroll
    for (int u = 0; u < W; ++u) y[u] = to_float(from_float<T>(zrow[i + u] * inv_r * (a.pre_gemma ? 1.f + wr[u] : wr[u])));
    if constexpr (VEC) {
      if (out) Vec4<T>::store(out + dst + i, y);
      if (a.out_f32) Vec4<float>::store(a.out_f32 + dst + i, y);
    } else {
      if (out) out[dst + i] = from_float<T>(y[0]);
      if (a.out_f32) a.out_f32[dst + i] = y[0];
    }
  }
}

// The same for rows of at most 1,024 x PER elements that allow 16-byte accesses: a thread keeps its (at most PER x 4)
// elements of a w_a and of the stream in registers, so the three passes touch neither shared memory (but for the two
// sums over the block) nor, after the first, global memory; the stream norm's weight is asked for in the first pass too.
template <typename T, int PER>
__global__ void __launch_bounds__(256) postnorm_add_norm_regs_kernel(SandwichArgs a) {
  pdl_wait();
  pdl_trigger();
  __shared__ float red[33];
  const int r = blockIdx.x;
  const int src_row = a.rows ? a.rows[r] : r;
  const size_t src = (size_t)src_row * a.hidden, dst = (size_t)r * a.hidden;
  const T* x = (const T*)a.x;
  const T* shared = (const T*)a.shared;
  float av[PER][4], zv[PER][4], wr[PER][4];
  int route[8];
  if (a.route_pos) {
#pragma unroll
    for (int j = 0; j < 8; ++j) route[j] = j < a.top_k ? a.route_pos[(size_t)src_row * a.top_k + j] : -1;
  }
  float ss = 0.f;
#pragma unroll
  for (int p = 0; p < PER; ++p) {
    const int i = (p * 256 + threadIdx.x) * 4;
#pragma unroll
    for (int u = 0; u < 4; ++u) av[p][u] = zv[p][u] = wr[p][u] = 0.f;
    if (i >= a.hidden) continue;
    float v[4], wa[4];
    Vec4<float>::load(a.residual + src + i, zv[p]);
    Vec4<float>::load(a.post_w + i, wa);
    if (a.pre_w) Vec4<float>::load(a.pre_w + i, wr[p]);
    if (a.route_pos) {
      v[0] = v[1] = v[2] = v[3] = 0.f;
      for (int j = 0; j < a.top_k; ++j) {  // route order
        const int q = j < 8 ? route[j] : a.route_pos[(size_t)src_row * a.top_k + j];
        if (q >= 0 && q < a.n_routes) {
          float y[4];
          Vec4<T>::load(x + (size_t)q * a.hidden + i, y);
#pragma unroll
          for (int u = 0; u < 4; ++u) v[u] += y[u];
        }
      }
      if (shared) {
        float y[4];
        Vec4<T>::load(shared + src + i, y);
#pragma unroll
        for (int u = 0; u < 4; ++u) v[u] += y[u];
      }
    } else {
      Vec4<T>::load(x + src + i, v);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      ss += v[u] * v[u];
      av[p][u] = v[u] * (a.post_gemma ? 1.f + wa[u] : wa[u]);
    }
  }
  ss = block_sum(ss, red);
  const float inv_a = rsqrtf(ss / (float)a.hidden + a.post_eps);
  float ss2 = 0.f;
#pragma unroll
  for (int p = 0; p < PER; ++p) {
    const int i = (p * 256 + threadIdx.x) * 4;
    if (i >= a.hidden) continue;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      zv[p][u] += av[p][u] * inv_a;
      ss2 += zv[p][u] * zv[p][u];
    }
    if (!a.rows) Vec4<float>::store(a.residual + src + i, zv[p]);
  }
  if (!a.pre_w) return;
  ss2 = block_sum(ss2, red);
  const float inv_r = rsqrtf(ss2 / (float)a.hidden + a.pre_eps);
  T* out = (T*)a.out;
#pragma unroll
  for (int p = 0; p < PER; ++p) {
    const int i = (p * 256 + threadIdx.x) * 4;
    if (i >= a.hidden) continue;
    float y[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) y[u] = to_float(from_float<T>(zv[p][u] * inv_r * (a.pre_gemma ? 1.f + wr[p][u] : wr[p][u])));
    if (out) Vec4<T>::store(out + dst + i, y);
    if (a.out_f32) Vec4<float>::store(a.out_f32 + dst + i, y);
  }
}

// One warp per (token, head).  x: [T, n_heads, x_stride] (XT), g: row t at g + t * g_stride, head h at + h * dim,
// out: [T, n_heads, out_stride] (T).  Columns past `dim` of a padded destination are left as they are.
template <typename XT, typename T>
__global__ void gated_heads_kernel(const XT* __restrict__ x, int x_stride, const T* __restrict__ g, long long g_stride,
                                   const float* __restrict__ norm_w, float eps, int act, T* __restrict__ out,
                                   int out_stride, int n_tokens, int n_heads, int dim) {
  pdl_wait();
  pdl_trigger();
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= (long long)n_tokens * n_heads) return;
  const int lane = threadIdx.x & 31;
  const long long t = w / n_heads;
  const int h = (int)(w % n_heads);
  const XT* xr = x + (size_t)w * x_stride;
  const T* gr = g + t * g_stride + (size_t)h * dim;
  T* o = out + (size_t)w * out_stride;
  float inv = 1.f;
  if (norm_w) {
    float ss = 0.f;
    for (int d = lane; d < dim; d += 32) {
      const float v = to_float(xr[d]);
      ss += v * v;
    }
    ss = warp_sum(ss);
    inv = rsqrtf(ss / (float)dim + eps);
  }
  for (int d = lane; d < dim; d += 32) {
    float v = to_float(xr[d]) * inv;
    if (norm_w) v *= norm_w[d];
    const float gv = to_float(gr[d]);
    const float s = 1.f / (1.f + expf(-gv));
    o[d] = from_float<T>(v * (act == FTK_GATE_SILU ? gv * s : s));
  }
}

// The same for heads of 8 x 2^k elements (k <= 5) whose rows allow 16-byte accesses: a thread takes eight consecutive
// elements, the TPR threads of a row sit side by side in a warp and add their squares by shuffles.
template <typename XT, int TPR>
__global__ void __launch_bounds__(256) gated_heads_vec_kernel(const XT* __restrict__ x, int x_stride,
                                                              const __nv_bfloat16* __restrict__ g, long long g_stride,
                                                              const float* __restrict__ norm_w, float eps, int act,
                                                              __nv_bfloat16* __restrict__ out, int out_stride,
                                                              int n_tokens, int n_heads) {
  pdl_wait();
  pdl_trigger();
  constexpr int dim = TPR * 8;
  const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) / TPR;
  const int d = (threadIdx.x % TPR) * 8;
  const bool ok = w < (long long)n_tokens * n_heads;
  const long long wr = ok ? w : 0;
  const long long t = wr / n_heads;
  const int h = (int)(wr % n_heads);
  float v[8], gv[8];
  if constexpr (sizeof(XT) == 4) {
    const float* xr = reinterpret_cast<const float*>(x) + (size_t)wr * x_stride + d;
    const float4 a = *reinterpret_cast<const float4*>(xr), b = *reinterpret_cast<const float4*>(xr + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else {
    const uint4 raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(x) + (size_t)wr * x_stride + d);
    const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int u = 0; u < 4; ++u) { const float2 f = __bfloat1622float2(p2[u]); v[2 * u] = f.x; v[2 * u + 1] = f.y; }
  }
  {
    const uint4 raw = *reinterpret_cast<const uint4*>(g + t * g_stride + (size_t)h * dim + d);
    const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int u = 0; u < 4; ++u) { const float2 f = __bfloat1622float2(p2[u]); gv[2 * u] = f.x; gv[2 * u + 1] = f.y; }
  }
  float inv = 1.f;
  if (norm_w) {
    float ss = 0.f;
#pragma unroll
    for (int u = 0; u < 8; ++u) ss += v[u] * v[u];
#pragma unroll
    for (int o = TPR / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    inv = rsqrtf(ss / (float)dim + eps);
  }
  uint4 res;
  __nv_bfloat162* r2 = reinterpret_cast<__nv_bfloat162*>(&res);
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    float y[2];
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      const int i = 2 * u + q;
      float val = v[i] * inv;
      if (norm_w) val *= norm_w[d + i];
      const float sg = 1.f / (1.f + expf(-gv[i]));
      y[q] = val * (act == FTK_GATE_SILU ? gv[i] * sg : sg);
    }
    r2[u] = __floats2bfloat162_rn(y[0], y[1]);
  }
  if (ok) *reinterpret_cast<uint4*>(out + (size_t)w * out_stride + d) = res;
}

__global__ void softcap_kernel(float* x, long long n, float cap) {
  pdl_wait();
  pdl_trigger();
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const float inv = 1.f / cap;
  for (; i < n; i += stride) x[i] = cap * tanhf(x[i] * inv);
}

}  // namespace ftk

using namespace ftk;

extern "C" int ftk_postnorm_add_norm(const void* x, int dtype, const int32_t* route_pos, int top_k, int n_routes,
                                     const void* shared, const float* post_w, float post_eps, int post_gemma,
                                     float* residual, const float* pre_w, float pre_eps, int pre_gemma, void* out,
                                     float* out_f32, const int32_t* rows, int n_rows, int hidden, void* stream) {
  FTK_REQUIRE(dtype_ok(dtype), "postnorm_add_norm: bad dtype %d", dtype);
  FTK_REQUIRE(n_rows >= 0 && hidden >= 1, "postnorm_add_norm: bad sizes");
  if (n_rows == 0) return 0;
  FTK_REQUIRE(x && post_w && residual, "postnorm_add_norm: null pointer");
  FTK_REQUIRE(!route_pos || (top_k >= 1 && n_routes >= 0), "postnorm_add_norm: bad route counts");
  FTK_REQUIRE(pre_w || (!out && !out_f32), "postnorm_add_norm: an output needs the weight of the stream's norm");
  FTK_REQUIRE(!pre_w || out || out_f32, "postnorm_add_norm: the stream's norm needs an output");
  FTK_REQUIRE(!rows || pre_w, "postnorm_add_norm: rows are picked for an output only");
  SandwichArgs a;
  a.x = x; a.route_pos = route_pos; a.top_k = top_k; a.n_routes = n_routes; a.shared = route_pos ? shared : nullptr;
  a.post_w = post_w; a.residual = residual; a.pre_w = pre_w; a.out = out; a.out_f32 = out_f32; a.rows = rows;
  a.n_rows = n_rows; a.hidden = hidden; a.post_eps = post_eps; a.pre_eps = pre_eps;
  a.post_gemma = post_gemma; a.pre_gemma = pre_gemma;
  const size_t smem = (size_t)2 * hidden * sizeof(float);
  FTK_REQUIRE(smem <= 200 * 1024, "postnorm_add_norm: rows of %d elements do not fit shared memory", hidden);
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  const bool vec = hidden % 8 == 0 && al16(x) && al16(shared) && al16(residual) && al16(post_w) && al16(pre_w) &&
                   al16(out) && al16(out_f32);
  auto go = [&](auto kern) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return FTK_LAUNCH(kern, n_rows, 256, smem, stream, a);
  };
  const int per = (hidden + 1023) / 1024;  // 16-byte pieces a thread of 256 holds of a row
  if (vec && per <= 8) {  // the row stays in registers
    const int P = per <= 1 ? 1 : per <= 2 ? 2 : per <= 4 ? 4 : 8;
    if (dtype == FTK_F32) {
      if (P == 1) FTK_LAUNCH((postnorm_add_norm_regs_kernel<float, 1>), n_rows, 256, 0, stream, a);
      else if (P == 2) FTK_LAUNCH((postnorm_add_norm_regs_kernel<float, 2>), n_rows, 256, 0, stream, a);
      else if (P == 4) FTK_LAUNCH((postnorm_add_norm_regs_kernel<float, 4>), n_rows, 256, 0, stream, a);
      else FTK_LAUNCH((postnorm_add_norm_regs_kernel<float, 8>), n_rows, 256, 0, stream, a);
    } else {
      if (P == 1) FTK_LAUNCH((postnorm_add_norm_regs_kernel<__nv_bfloat16, 1>), n_rows, 256, 0, stream, a);
      else if (P == 2) FTK_LAUNCH((postnorm_add_norm_regs_kernel<__nv_bfloat16, 2>), n_rows, 256, 0, stream, a);
      else if (P == 4) FTK_LAUNCH((postnorm_add_norm_regs_kernel<__nv_bfloat16, 4>), n_rows, 256, 0, stream, a);
      else FTK_LAUNCH((postnorm_add_norm_regs_kernel<__nv_bfloat16, 8>), n_rows, 256, 0, stream, a);
    }
  } else if (dtype == FTK_F32) {
    if (vec) go(postnorm_add_norm_kernel<float, true>);
    else go(postnorm_add_norm_kernel<float, false>);
  } else {
    if (vec) go(postnorm_add_norm_kernel<__nv_bfloat16, true>);
    else go(postnorm_add_norm_kernel<__nv_bfloat16, false>);
  }
  FTK_LAUNCH_CHECK("postnorm_add_norm");
  return 0;
}

extern "C" int ftk_gated_heads(const void* x, int x_f32, int x_stride, const void* gates, long long gate_stride,
                               const float* norm_w, float eps, int act, void* out, int out_stride, int dtype,
                               int n_tokens, int n_heads, int dim, void* stream) {
  FTK_REQUIRE(dtype_ok(dtype), "gated_heads: bad dtype %d", dtype);
  FTK_REQUIRE(act == FTK_GATE_SIGMOID || act == FTK_GATE_SILU, "gated_heads: unknown gate %d", act);
  FTK_REQUIRE(n_tokens >= 0 && n_heads >= 1 && dim >= 1 && x_stride >= dim && out_stride >= dim &&
                  gate_stride >= (long long)n_heads * dim,
              "gated_heads: bad sizes");
  if (n_tokens == 0) return 0;
  FTK_REQUIRE(x && gates && out, "gated_heads: null pointer");
  const long long rows = (long long)n_tokens * n_heads;
  const int tpr = dim / 8;
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (dtype == FTK_BF16 && dim % 8 == 0 && tpr <= 32 && (tpr & (tpr - 1)) == 0 && x_stride % 8 == 0 && out_stride % 8 == 0 &&
      gate_stride % 8 == 0 && al16(x) && al16(gates) && al16(out) && (!norm_w || al16(norm_w))) {
    const long long threads = rows * tpr;
    const unsigned blocks = (unsigned)((threads + 255) / 256);
    const __nv_bfloat16* g = (const __nv_bfloat16*)gates;
    __nv_bfloat16* o = (__nv_bfloat16*)out;
#define FTK_GH(XT, N) FTK_LAUNCH((gated_heads_vec_kernel<XT, N>), blocks, 256, 0, stream, (const XT*)x, x_stride, g, gate_stride, \
                                 norm_w, eps, act, o, out_stride, n_tokens, n_heads)
#define FTK_GH_ALL(XT)                                                                                        \
    (tpr == 1 ? FTK_GH(XT, 1) : tpr == 2 ? FTK_GH(XT, 2) : tpr == 4 ? FTK_GH(XT, 4) : tpr == 8 ? FTK_GH(XT, 8) \
     : tpr == 16 ? FTK_GH(XT, 16) : FTK_GH(XT, 32))
    if (x_f32) FTK_GH_ALL(float);
    else FTK_GH_ALL(__nv_bfloat16);
#undef FTK_GH_ALL
#undef FTK_GH
    FTK_LAUNCH_CHECK("gated_heads");
    return 0;
  }
  const int warps = 8;
  const unsigned blocks = (unsigned)((rows + warps - 1) / warps);
  if (dtype == FTK_F32) {
    FTK_LAUNCH((gated_heads_kernel<float, float>), blocks, warps * 32, 0, stream, (const float*)x, x_stride,
               (const float*)gates, gate_stride, norm_w, eps, act, (float*)out, out_stride, n_tokens, n_heads, dim);
  } else if (x_f32) {
    FTK_LAUNCH((gated_heads_kernel<float, __nv_bfloat16>), blocks, warps * 32, 0, stream, (const float*)x, x_stride,
               (const __nv_bfloat16*)gates, gate_stride, norm_w, eps, act, (__nv_bfloat16*)out, out_stride, n_tokens,
               n_heads, dim);
  } else {
    FTK_LAUNCH((gated_heads_kernel<__nv_bfloat16, __nv_bfloat16>), blocks, warps * 32, 0, stream,
               (const __nv_bfloat16*)x, x_stride, (const __nv_bfloat16*)gates, gate_stride, norm_w, eps, act,
               (__nv_bfloat16*)out, out_stride, n_tokens, n_heads, dim);
  }
  FTK_LAUNCH_CHECK("gated_heads");
  return 0;
}

extern "C" int ftk_softcap_f32(float* x, long long n, float cap, void* stream) {
  FTK_REQUIRE(n >= 0 && cap > 0.f, "softcap: bad arguments");
  if (n == 0) return 0;
  FTK_REQUIRE(x, "softcap: null pointer");
  const unsigned blocks = (unsigned)((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
  FTK_LAUNCH(softcap_kernel, blocks, 256, 0, stream, x, n, cap);
  FTK_LAUNCH_CHECK("softcap");
  return 0;
}
