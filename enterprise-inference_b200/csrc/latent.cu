// Latent attention (B200_MIXER_LATENT): what surrounds the paged attention kernel.
//
// Per token the fused projection gives queries (per head `dim` plain + `rot_dim` rotated dimensions), a latent of kv_rank
// dimensions and one rotated key part shared by all heads.  Only [normed latent | rotated key part] is cached.  A head's
// plain key is W_uk c, so q_plain . (W_uk c) = (W_uk^T q_plain) . c: the scores are taken against the cached rows directly
// with q' = [W_uk^T q_plain | rotated q] (one kv head of kv_rank + rot_dim dimensions), the weighted sum of the cached
// latents (the row's first kv_rank entries are the "values") is expanded by W_uv afterwards.
//
//  * latent_prep: RMS norm of the latent with its weight, rotation of the shared key part and of every head's rotated query
//    part (interleaved pairs, fp32 cos|sin table), cache append, rotated query parts into the fp32 query rows;
//  * head_linear: y[t][h] = W[h] x[t][h] for every head at once, strided rows in and out, fp32 accumulation, optional
//    sigmoid gate on the output (the output gate of the mixer reads the same input as the projections).
#include "common.cuh"

namespace b200 {
namespace {

template <typename AT> __device__ __forceinline__ float ldx(const AT* p, int64_t i);
template <> __device__ __forceinline__ float ldx<float>(const float* p, int64_t i) { return p[i]; }
template <> __device__ __forceinline__ float ldx<__nv_bfloat16>(const __nv_bfloat16* p, int64_t i) { return __bfloat162float(p[i]); }
template <typename AT> __device__ __forceinline__ void stx(AT* p, int64_t i, float v);
template <> __device__ __forceinline__ void stx<float>(float* p, int64_t i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void stx<__nv_bfloat16>(__nv_bfloat16* p, int64_t i, float v) { p[i] = __float2bfloat16_rn(v); }

// one CTA (128 threads) per row
template <typename AT>
__global__ void __launch_bounds__(128)
latent_prep_kernel(const AT* __restrict__ qkv, int64_t ld, const float* __restrict__ norm_w, const int32_t* __restrict__ positions,
                   const int32_t* __restrict__ slots, const float* __restrict__ rot, int rot_dims, int64_t max_pos,
                   float* __restrict__ qfull, AT* __restrict__ cache, int heads, int dim, int rot_dim, int kv_rank, float eps) {
  __shared__ float red[4];
  pdl_wait();
  pdl_launch_dependents();
  const int64_t t = blockIdx.x;
  const AT* row = qkv + t * ld;
  const int qh = dim + rot_dim, krow = kv_rank + rot_dim;
  const AT* dkv = row + (int64_t)heads * qh;
  int pos = positions[t];
  pos = pos < 0 ? 0 : (pos >= max_pos ? (int)max_pos - 1 : pos);
  const int half = rot_dims >> 1;
  const float* cs = rot ? rot + (int64_t)pos * 2 * half : nullptr;
  float ss = 0.f;
  for (int c = threadIdx.x; c < kv_rank; c += 128) {
    const float v = ldx<AT>(dkv, c);
    ss = fmaf(v, v, ss);
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  const float inv = rsqrtf(((red[0] + red[1]) + (red[2] + red[3])) / (float)kv_rank + eps);
  AT* dst = cache + (int64_t)slots[t] * krow;
  for (int c = threadIdx.x; c < kv_rank; c += 128) stx<AT>(dst, c, ldx<AT>(dkv, c) * inv * norm_w[c]);
  // rotated parts: index e over (heads + 1) vectors of rot_dim entries; vector `heads` is the shared key part
  for (int e = threadIdx.x; e < (heads + 1) * rot_dim; e += 128) {
    const int hv = e / rot_dim, i = e % rot_dim;
    const AT* src = hv < heads ? row + (int64_t)hv * qh + dim : dkv + kv_rank;
    float v = ldx<AT>(src, i);
    if (cs && i < 2 * half) {
      const float o = ldx<AT>(src, i ^ 1), c = cs[i >> 1], s = cs[half + (i >> 1)];
      v = (i & 1) ? fmaf(v, c, o * s) : fmaf(v, c, -o * s);
    }
    if (hv < heads) qfull[(t * heads + hv) * krow + kv_rank + i] = v;
    else stx<AT>(dst, kv_rank + i, v);
  }
}

// CTA = (tile of kHlRows rows, head).  The rows' inputs are staged in shared memory as fp32; warp w owns outputs w, w + 8,
// ...; a lane strides the inner dimension for all rows at once.
constexpr int kHlRows = 16;
template <typename AT, typename YT>
__global__ void __launch_bounds__(256)
head_linear_kernel(const AT* __restrict__ x, int64_t ldx_, int x_hs, const __nv_bfloat16* __restrict__ w, YT* __restrict__ y, int64_t ldy,
                   int y_hs, const AT* __restrict__ gate, int64_t ldg, int g_hs, int T, int n_out, int k) {
  extern __shared__ float xs[];   // [kHlRows][k]
  pdl_wait();
  pdl_launch_dependents();
  const int t0 = blockIdx.x * kHlRows, h = blockIdx.y, nr = min(kHlRows, T - t0);
  for (int i = threadIdx.x; i < kHlRows * k; i += 256) {
    const int r = i / k, c = i % k;
    xs[i] = r < nr ? ldx<AT>(x, (int64_t)(t0 + r) * ldx_ + (int64_t)h * x_hs + c) : 0.f;
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const __nv_bfloat16* wh = w + (int64_t)h * n_out * k;
  for (int o = warp; o < n_out; o += 8) {
    const __nv_bfloat16* wr = wh + (int64_t)o * k;
    float acc[kHlRows];
#pragma unroll
    for (int r = 0; r < kHlRows; ++r) acc[r] = 0.f;
    for (int c = lane; c < k; c += 32) {
      const float wv = __bfloat162float(wr[c]);
#pragma unroll
      for (int r = 0; r < kHlRows; ++r) acc[r] = fmaf(wv, xs[r * k + c], acc[r]);
    }
#pragma unroll
    for (int r = 0; r < kHlRows; ++r) {
      float v = warp_sum(acc[r]);
      if (lane == 0 && r < nr) {
        if (gate) v *= 1.0f / (1.0f + expf(-ldx<AT>(gate, (int64_t)(t0 + r) * ldg + (int64_t)h * g_hs + o)));
        stx<YT>(y, (int64_t)(t0 + r) * ldy + (int64_t)h * y_hs + o, v);
      }
    }
  }
}

}  // namespace

int latent_prep(bool f32, const void* qkv, int64_t ld, const float* norm_w, const int32_t* positions, const int32_t* slots,
                const float* rot, int rot_dims, int64_t max_pos, float* qfull, void* cache, int T, int heads, int dim, int rot_dim,
                int kv_rank, float eps, cudaStream_t s) {
  if (T == 0) return B200_OK;
  B200_REQUIRE(rot_dims >= 0 && rot_dims <= rot_dim && rot_dims % 2 == 0, B200_ERR_INVALID, "latent_prep: %d of %d dimensions rotate",
               rot_dims, rot_dim);
  if (f32)
    B200_CUDA(launch(latent_prep_kernel<float>, dim3(T), dim3(128), (size_t)0, s, (const float*)qkv, ld, norm_w, positions, slots, rot,
                     rot ? rot_dims : 0, max_pos, qfull, (float*)cache, heads, dim, rot_dim, kv_rank, eps));
  else
    B200_CUDA(launch(latent_prep_kernel<__nv_bfloat16>, dim3(T), dim3(128), (size_t)0, s, (const __nv_bfloat16*)qkv, ld, norm_w, positions,
                     slots, rot, rot ? rot_dims : 0, max_pos, qfull, (__nv_bfloat16*)cache, heads, dim, rot_dim, kv_rank, eps));
  return B200_OK;
}

template <typename AT, typename YT>
static int head_linear_t(const void* x, int64_t ldx_, int x_hs, const __nv_bfloat16* w, void* y, int64_t ldy, int y_hs, const void* gate,
                         int64_t ldg, int g_hs, int T, int heads, int n_out, int k, cudaStream_t s) {
  const size_t smem = (size_t)kHlRows * k * 4;
  B200_REQUIRE(smem <= 200 * 1024, B200_ERR_UNSUPPORTED, "head_linear: inner size %d does not fit shared memory", k);
  static bool done[64] = {};
  if (smem > 48 * 1024) B200_CUDA(ensure_dynamic_smem(head_linear_kernel<AT, YT>, 200 * 1024, done));
  B200_CUDA(launch(head_linear_kernel<AT, YT>, dim3((T + kHlRows - 1) / kHlRows, heads), dim3(256), smem, s, (const AT*)x, ldx_, x_hs, w,
                   (YT*)y, ldy, y_hs, (const AT*)gate, ldg, g_hs, T, n_out, k));
  return B200_OK;
}

// x, gate: activation type (fp32 when f32, else bf16); y: fp32 when y_f32, else the activation type
int head_linear(bool f32, bool y_f32, const void* x, int64_t ldx_, int x_hs, const __nv_bfloat16* w, void* y, int64_t ldy, int y_hs,
                const void* gate, int64_t ldg, int g_hs, int T, int heads, int n_out, int k, cudaStream_t s) {
  if (T == 0) return B200_OK;
  if (f32) return head_linear_t<float, float>(x, ldx_, x_hs, w, y, ldy, y_hs, gate, ldg, g_hs, T, heads, n_out, k, s);
  if (y_f32) return head_linear_t<__nv_bfloat16, float>(x, ldx_, x_hs, w, y, ldy, y_hs, gate, ldg, g_hs, T, heads, n_out, k, s);
  return head_linear_t<__nv_bfloat16, __nv_bfloat16>(x, ldx_, x_hs, w, y, ldy, y_hs, gate, ldg, g_hs, T, heads, n_out, k, s);
}

}  // namespace b200
