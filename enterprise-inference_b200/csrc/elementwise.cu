// The small ops of the decode step: embedding gather (a1), (add+)RMSNorm (a2), RoPE + KV append
// (a4+a5), SiLU*mul (a8), greedy argmax (a10).  All are latency/launch bound at decode sizes;
// their bytes are noise next to the weight stream, so the design goal is: vectorised 16-byte
// accesses, one pass over the data, rounding points identical to oracle/decode_oracle.py R1/R3/R5/R6.
#include <algorithm>

#include "common.cuh"

namespace b200 {

namespace {

// ---------------------------------------------------------------------------------------
// (a1) embedding
// ---------------------------------------------------------------------------------------
// A negative id -(j+1) stands for "the token the previous step chose for its logit row j", still on the device
// (prev): a host that schedules step n+1 while step n runs does not know that token yet.
__device__ __forceinline__ int resolve_id(int id, int vocab, const int32_t* prev, int n_prev) {
  if (id < 0 && prev != nullptr && -id - 1 < n_prev) id = prev[-id - 1];
  return id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);  // ids are validated on the host; clamp, never fault
}

__global__ void __launch_bounds__(128)
embed_kernel(const int32_t* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
             __nv_bfloat16* __restrict__ out, int hidden, int vocab, const int32_t* prev, int n_prev) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int id = resolve_id(ids[t], vocab, prev, n_prev);
  const uint4* src = reinterpret_cast<const uint4*>(table + (int64_t)id * hidden);
  uint4* dst = reinterpret_cast<uint4*>(out + (int64_t)t * hidden);
  for (int c = threadIdx.x; c < hidden / 8; c += blockDim.x) dst[c] = __ldg(src + c);
}

// ---------------------------------------------------------------------------------------
// (a2) RMSNorm / fused add + RMSNorm.  One CTA per token row, the row lives in registers.
//   s = x (+ res) in fp32; res' = bf16(s); var over UNROUNDED s; n = bf16(s / sqrt(var+eps));
//   y = bf16(n * w)                                   [V22] vllm/ir/ops/layernorm.py:10-21,40-58
// ---------------------------------------------------------------------------------------
// The sum of squares is taken in a fixed order that the linears' fused-norm path reproduces exactly (gemm_tc.cu,
// finalize4<kResidual> / norm_b_tiles): per 128-wide slab, lane l squares its 4 values 4l..4l+3 in order (fma chain),
// the warp tree (xor 16, 8, 4, 2, 1) adds the lanes, and the slab sums are added in ascending slab order.
constexpr int kNormThreads = 256;
constexpr int kNormWarps = kNormThreads / 32;
constexpr int kNormMaxSlabs = 8;  // per warp: hidden <= 8 * 8 * 128 = 8192

template <bool HAS_RES>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* res, const __nv_bfloat16* __restrict__ w,
               __nv_bfloat16* y, int hidden, float eps) {
  __shared__ float part[kNormWarps * kNormMaxSlabs];
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nslab = hidden >> 7;
  const uint2* xr = reinterpret_cast<const uint2*>(x + (int64_t)t * hidden);
  uint2* rr = HAS_RES ? reinterpret_cast<uint2*>(res + (int64_t)t * hidden) : nullptr;
  float v[kNormMaxSlabs][4];
#pragma unroll
  for (int i = 0; i < kNormMaxSlabs; ++i) {
    const int slab = warp + i * kNormWarps;
    if (slab < nslab) {
      const int c = slab * 32 + lane;   // 8-byte chunk index
      const uint2 a = xr[c];
      if (HAS_RES) {
        const uint2 b = rr[c];
        v[i][0] = bf16lo(a.x) + bf16lo(b.x);
        v[i][1] = bf16hi(a.x) + bf16hi(b.x);
        v[i][2] = bf16lo(a.y) + bf16lo(b.y);
        v[i][3] = bf16hi(a.y) + bf16hi(b.y);
        rr[c] = make_uint2(pack_bf16(v[i][0], v[i][1]), pack_bf16(v[i][2], v[i][3]));
      } else {
        v[i][0] = bf16lo(a.x);
        v[i][1] = bf16hi(a.x);
        v[i][2] = bf16lo(a.y);
        v[i][3] = bf16hi(a.y);
      }
      float ss = fmaf(v[i][0], v[i][0], 0.f);
      ss = fmaf(v[i][1], v[i][1], ss);
      ss = fmaf(v[i][2], v[i][2], ss);
      ss = fmaf(v[i][3], v[i][3], ss);
      ss = warp_sum(ss);
      if (lane == 0) part[slab] = ss;
    }
  }
  __syncthreads();
  float tot = 0.f;
  for (int i = 0; i < nslab; ++i) tot += part[i];
  const float r = 1.0f / sqrtf(tot / (float)hidden + eps);
  const uint2* wr = reinterpret_cast<const uint2*>(w);
  uint2* yr = reinterpret_cast<uint2*>(y + (int64_t)t * hidden);
#pragma unroll
  for (int i = 0; i < kNormMaxSlabs; ++i) {
    const int slab = warp + i * kNormWarps;
    if (slab < nslab) {
      const int c = slab * 32 + lane;
      const uint2 wq = __ldg(wr + c);
      const float n0 = round_bf16(v[i][0] * r), n1 = round_bf16(v[i][1] * r);
      const float n2 = round_bf16(v[i][2] * r), n3 = round_bf16(v[i][3] * r);
      yr[c] = make_uint2(pack_bf16(n0 * bf16lo(wq.x), n1 * bf16hi(wq.x)), pack_bf16(n2 * bf16lo(wq.y), n3 * bf16hi(wq.y)));
    }
  }
}

// Embedding rows into the fp32 residual stream: sres[t] = float(table[ids[t]]), ssq[t][slab] in the order above.
__global__ void __launch_bounds__(kNormThreads)
embed_stream_kernel(const int32_t* __restrict__ ids, const __nv_bfloat16* __restrict__ table, float* __restrict__ sres,
                    float* __restrict__ ssq, int hidden, int vocab, const int32_t* prev, int n_prev) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nslab = hidden >> 7;
  const int id = resolve_id(ids[t], vocab, prev, n_prev);
  const uint2* src = reinterpret_cast<const uint2*>(table + (int64_t)id * hidden);
  float4* dst = reinterpret_cast<float4*>(sres + (int64_t)t * hidden);
  for (int slab = warp; slab < nslab; slab += kNormWarps) {
    const uint2 a = __ldg(src + slab * 32 + lane);
    const float4 f = make_float4(bf16lo(a.x), bf16hi(a.x), bf16lo(a.y), bf16hi(a.y));
    dst[slab * 32 + lane] = f;
    float ss = fmaf(f.x, f.x, 0.f);
    ss = fmaf(f.y, f.y, ss);
    ss = fmaf(f.z, f.z, ss);
    ss = fmaf(f.w, f.w, ss);
    ss = warp_sum(ss);
    if (lane == 0) ssq[(int64_t)t * nslab + slab] = ss;
  }
}

// Stream rows -> normalised bf16 rows (the consumer side of the folded norm as a kernel of its own, for consumers
// that would re-normalise the same rows in too many CTAs: lm_head over many logit rows).
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_stream_kernel(const float* __restrict__ sres, const float* __restrict__ ssq, const int32_t* __restrict__ rows,
                      const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y, int hidden, float eps) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int row = rows ? rows[t] : t;
  const int nslab = hidden >> 7;
  float tot = 0.f;
  for (int i = 0; i < nslab; ++i) tot += __ldcg(ssq + (int64_t)row * nslab + i);
  const float r = 1.0f / sqrtf(tot / (float)hidden + eps);
  const float4* sr = reinterpret_cast<const float4*>(sres + (int64_t)row * hidden);
  const uint2* wr = reinterpret_cast<const uint2*>(w);
  uint2* yr = reinterpret_cast<uint2*>(y + (int64_t)t * hidden);
  for (int c = threadIdx.x; c < hidden / 4; c += kNormThreads) {
    const float4 s4 = __ldcg(sr + c);
    const uint2 wq = __ldg(wr + c);
    const float n0 = round_bf16(s4.x * r), n1 = round_bf16(s4.y * r), n2 = round_bf16(s4.z * r), n3 = round_bf16(s4.w * r);
    yr[c] = make_uint2(pack_bf16(n0 * bf16lo(wq.x), n1 * bf16hi(wq.x)), pack_bf16(n2 * bf16lo(wq.y), n3 * bf16hi(wq.y)));
  }
}

// ---------------------------------------------------------------------------------------
// (a4+a5) NeoX RoPE in bf16 arithmetic on q and k heads, then K/V rows into the paged cache.
// grid (token, head), 64 threads: thread i owns the pair (i, i+64).
// cache layout per layer: [block][kv head][block_size][128].
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(64)
rope_kv_kernel(__nv_bfloat16* qkv, const int32_t* __restrict__ positions, const int32_t* __restrict__ slots,
               const __nv_bfloat16* __restrict__ cos_sin, __nv_bfloat16* kc, __nv_bfloat16* vc, int hq, int hkv,
               int block_size) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x, head = blockIdx.y, i = threadIdx.x;
  const int row_w = (hq + 2 * hkv) * kHeadDim;
  __nv_bfloat16* hp = qkv + (int64_t)t * row_w + head * kHeadDim;
  const int slot = slots[t];
  if (head < hq + hkv) {
    const int pos = positions[t];
    const __nv_bfloat16* cs = cos_sin + (int64_t)pos * kHeadDim;
    const float c = __bfloat162float(cs[i]), s = __bfloat162float(cs[i + 64]);
    const float x1 = __bfloat162float(hp[i]), x2 = __bfloat162float(hp[i + 64]);
    // every elementwise op rounds to bf16 (R3)
    const float o1 = round_bf16(round_bf16(x1 * c) - round_bf16(x2 * s));
    const float o2 = round_bf16(round_bf16(x2 * c) + round_bf16(x1 * s));
    if (head < hq) {
      hp[i] = __float2bfloat16_rn(o1);
      hp[i + 64] = __float2bfloat16_rn(o2);
    } else if (slot >= 0) {
      const int kvh = head - hq;
      const int64_t blk = slot / block_size, off = slot % block_size;
      __nv_bfloat16* dst = kc + ((blk * hkv + kvh) * block_size + off) * kHeadDim;
      dst[i] = __float2bfloat16_rn(o1);
      dst[i + 64] = __float2bfloat16_rn(o2);
    }
  } else if (slot >= 0) {
    const int kvh = head - hq - hkv;
    const int64_t blk = slot / block_size, off = slot % block_size;
    __nv_bfloat16* dst = vc + ((blk * hkv + kvh) * block_size + off) * kHeadDim;
    dst[i] = hp[i];
    dst[i + 64] = hp[i + 64];
  }
}

// ---------------------------------------------------------------------------------------
// (a8) SiLU*mul: a = bf16(bf16(silu(g)) * u)             [V22] activation.py:137-141
// ---------------------------------------------------------------------------------------

__global__ void __launch_bounds__(256)
silu_mul_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, int inter, int64_t total_chunks) {
  pdl_wait();
  pdl_launch_dependents();
  const int cpr = inter >> 3;  // chunks per row
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total_chunks;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = idx / cpr;
    const int c = (int)(idx % cpr);
    const uint4 g = *reinterpret_cast<const uint4*>(gu + t * 2 * inter + c * 8);
    const uint4 u = *reinterpret_cast<const uint4*>(gu + t * 2 * inter + inter + c * 8);
    const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      o[j] = pack_bf16(silu_to_bf16(bf16lo(gw[j])) * bf16lo(uw[j]), silu_to_bf16(bf16hi(gw[j])) * bf16hi(uw[j]));
    *reinterpret_cast<uint4*>(out + t * inter + c * 8) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// ---------------------------------------------------------------------------------------
// (a10) greedy argmax per row, fp32 compare, ties -> lowest index.  [V22] sampler.py:90-91,235-236
// ---------------------------------------------------------------------------------------
constexpr int kArgmaxThreads = 1024;

__device__ __forceinline__ void take(float& bv, int& bi, float v, int i) {
  if (v > bv || (v == bv && i < bi)) {
    bv = v;
    bi = i;
  }
}

__global__ void __launch_bounds__(kArgmaxThreads)
argmax_kernel(const __nv_bfloat16* __restrict__ logits, int64_t ld, int vocab, int index_offset,
              int32_t* __restrict__ out_ids, float* __restrict__ out_max) {
  __shared__ float sv[kArgmaxThreads / 32];
  __shared__ int si[kArgmaxThreads / 32];
  pdl_wait();
  pdl_launch_dependents();
  const __nv_bfloat16* row = logits + (int64_t)blockIdx.x * ld;
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  const int nchunk = vocab >> 3;
  for (int c = threadIdx.x; c < nchunk; c += kArgmaxThreads) {
    const uint4 q = *reinterpret_cast<const uint4*>(row + c * 8);
    const uint32_t qw[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      take(bv, bi, bf16lo(qw[j]), c * 8 + 2 * j);
      take(bv, bi, bf16hi(qw[j]), c * 8 + 2 * j + 1);
    }
  }
  for (int i = nchunk * 8 + threadIdx.x; i < vocab; i += kArgmaxThreads) take(bv, bi, __bfloat162float(row[i]), i);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    take(bv, bi, ov, oi);
  }
  if ((threadIdx.x & 31) == 0) {
    sv[threadIdx.x >> 5] = bv;
    si[threadIdx.x >> 5] = bi;
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    bv = sv[threadIdx.x];
    bi = si[threadIdx.x];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      take(bv, bi, ov, oi);
    }
    if (threadIdx.x == 0) {
      out_ids[blockIdx.x] = bi + index_offset;
      if (out_max) out_max[blockIdx.x] = bv;
    }
  }
}

// ---------------------------------------------------------------------------------------
// (a0) device-side advance of pure-decode rows: the sampled token becomes the next input, position
// and context grow by one, the slot follows the block table.  Lets a caller run several decode
// steps without a host round trip (inputs stay resident in HBM).
// ---------------------------------------------------------------------------------------
__global__ void advance_rows_kernel(int32_t* ids, int32_t* positions, int32_t* slots, int32_t* ctx_lens,
                                    const int32_t* __restrict__ block_table, int bt_stride,
                                    const int32_t* __restrict__ row_to_seq, const int32_t* __restrict__ sampled, int n,
                                    int block_size) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n) return;
  const int p = positions[t] + 1;
  const int seq = row_to_seq ? row_to_seq[t] : t;
  ids[t] = sampled[t];
  positions[t] = p;
  ctx_lens[t] = p + 1;
  slots[t] = block_table[(int64_t)seq * bt_stride + p / block_size] * block_size + p % block_size;
}


// ---------------------------------------------------------------------------------------
// fp32 residual stream of layer-list models: x[t] = float(table[id]) * scale.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128)
embed_scaled_kernel(const int32_t* __restrict__ ids, const __nv_bfloat16* __restrict__ table, float* __restrict__ out,
                    int width, int vocab, float scale, const int32_t* prev, int n_prev) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int id = resolve_id(ids[t], vocab, prev, n_prev);
  const __nv_bfloat16* src = table + (int64_t)id * width;
  float* dst = out + (int64_t)t * width;
  for (int c = threadIdx.x; c < width; c += blockDim.x) dst[c] = __bfloat162float(src[c]) * scale;
}

// ---------------------------------------------------------------------------------------
// Layer norm without bias over an fp32 residual stream, with the sandwich form fused: one CTA per row,
//   (1) y given:   x += (y - mean(y)) / sqrt(var(y) + eps) * w_post   (var = mean of squared deviations; y is either an
//                  activation row or the sum, in a fixed order, of n_parts fp32 partial rows)
//   (2) w_next given: out = (x - mean(x)) / sqrt(var(x) + eps) * w_next, the input of the next sublayer.
// `rows` (nullable) picks the stream rows to read (the logit rows before the output projection).  All arithmetic fp32;
// the row is staged in shared memory, statistics are two-pass.
// ---------------------------------------------------------------------------------------
constexpr int kLnThreads = 256;

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();   // red may still be read from the previous call
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = 0.f;
  for (int i = 0; i < nw; ++i) r += red[i];   // same order in every thread
  return r;
}

template <typename AT> __device__ __forceinline__ float act_load(const AT* p, int64_t i);
template <> __device__ __forceinline__ float act_load<float>(const float* p, int64_t i) { return p[i]; }
template <> __device__ __forceinline__ float act_load<__nv_bfloat16>(const __nv_bfloat16* p, int64_t i) { return __bfloat162float(p[i]); }
template <typename AT> __device__ __forceinline__ void act_store(AT* p, int64_t i, float v);
template <> __device__ __forceinline__ void act_store<float>(float* p, int64_t i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void act_store<__nv_bfloat16>(__nv_bfloat16* p, int64_t i, float v) { p[i] = __float2bfloat16_rn(v); }

// four consecutive activations (width % 4 == 0, 16-byte aligned fp32 rows / 8-byte aligned bf16 rows)
template <typename AT> __device__ __forceinline__ float4 act_load4(const AT* p, int64_t i);
template <> __device__ __forceinline__ float4 act_load4<float>(const float* p, int64_t i) { return *reinterpret_cast<const float4*>(p + i); }
template <> __device__ __forceinline__ float4 act_load4<__nv_bfloat16>(const __nv_bfloat16* p, int64_t i) {
  const uint2 v = *reinterpret_cast<const uint2*>(p + i);
  return make_float4(bf16lo(v.x), bf16hi(v.x), bf16lo(v.y), bf16hi(v.y));
}
template <typename AT> __device__ __forceinline__ void act_store4(AT* p, int64_t i, float4 v);
template <> __device__ __forceinline__ void act_store4<float>(float* p, int64_t i, float4 v) { *reinterpret_cast<float4*>(p + i) = v; }
template <> __device__ __forceinline__ void act_store4<__nv_bfloat16>(__nv_bfloat16* p, int64_t i, float4 v) {
  *reinterpret_cast<uint2*>(p + i) = make_uint2(pack_bf16(v.x, v.y), pack_bf16(v.z, v.w));
}

// VEC = 4: width % 4 == 0, every access is 4 elements wide; VEC = 1: any width.  The order of every sum over the row is the
// same function of (width, VEC) for every row, so a row's result does not depend on the step it is part of.
template <typename AT, int VEC>
__global__ void __launch_bounds__(kLnThreads)
layernorm_stream_kernel(float* x, const AT* __restrict__ y, const float* __restrict__ yparts, int n_parts,
                        const float* __restrict__ w_post, const float* __restrict__ w_next, AT* __restrict__ out,
                        const int32_t* __restrict__ rows, int width, float eps) {
  extern __shared__ __align__(16) float ln_row[];
  __shared__ float red[kLnThreads / 32];
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int64_t xrow = rows ? rows[t] : t;
  const int64_t xr = xrow * width;
  const float inv_w = 1.0f / (float)width;
  const int step = blockDim.x * VEC;
  if (y != nullptr || yparts != nullptr) {
    float sum = 0.f;
    for (int c = threadIdx.x * VEC; c < width; c += step) {
      if constexpr (VEC == 4) {
        float4 v;
        if (y != nullptr) {
          v = act_load4<AT>(y, xr + c);
        } else {
          v = make_float4(0.f, 0.f, 0.f, 0.f);
          for (int p = 0; p < n_parts; ++p) {
            const float4 q = *reinterpret_cast<const float4*>(yparts + (xrow * n_parts + p) * width + c);
            v.x += q.x; v.y += q.y; v.z += q.z; v.w += q.w;
          }
        }
        *reinterpret_cast<float4*>(ln_row + c) = v;
        sum += (v.x + v.y) + (v.z + v.w);
      } else {
        float v;
        if (y != nullptr) {
          v = act_load<AT>(y, xr + c);
        } else {
          v = 0.f;
          for (int p = 0; p < n_parts; ++p) v += yparts[(xrow * n_parts + p) * width + c];
        }
        ln_row[c] = v;
        sum += v;
      }
    }
    const float mean = block_sum(sum, red) * inv_w;
    float sq = 0.f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
      const float d = ln_row[c] - mean;
      sq = fmaf(d, d, sq);
    }
    const float rstd = 1.0f / sqrtf(block_sum(sq, red) * inv_w + eps);
    for (int c = threadIdx.x * VEC; c < width; c += step) {
      if constexpr (VEC == 4) {
        const float4 xo = *reinterpret_cast<const float4*>(x + xr + c), wv = *reinterpret_cast<const float4*>(w_post + c);
        const float4 l = *reinterpret_cast<const float4*>(ln_row + c);
        const float4 v = make_float4(xo.x + (l.x - mean) * rstd * wv.x, xo.y + (l.y - mean) * rstd * wv.y,
                                     xo.z + (l.z - mean) * rstd * wv.z, xo.w + (l.w - mean) * rstd * wv.w);
        *reinterpret_cast<float4*>(x + xr + c) = v;
        *reinterpret_cast<float4*>(ln_row + c) = v;
      } else {
        const float v = x[xr + c] + (ln_row[c] - mean) * rstd * w_post[c];
        x[xr + c] = v;
        ln_row[c] = v;
      }
    }
  } else {
    for (int c = threadIdx.x * VEC; c < width; c += step) {
      if constexpr (VEC == 4) *reinterpret_cast<float4*>(ln_row + c) = *reinterpret_cast<const float4*>(x + xr + c);
      else ln_row[c] = x[xr + c];
    }
  }
  if (w_next == nullptr) return;
  __syncthreads();   // the sums below read elements other threads staged
  float sum = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) sum += ln_row[c];
  const float mean = block_sum(sum, red) * inv_w;
  float sq = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float d = ln_row[c] - mean;
    sq = fmaf(d, d, sq);
  }
  const float rstd = 1.0f / sqrtf(block_sum(sq, red) * inv_w + eps);
  for (int c = threadIdx.x * VEC; c < width; c += step) {
    if constexpr (VEC == 4) {
      const float4 l = *reinterpret_cast<const float4*>(ln_row + c), wv = *reinterpret_cast<const float4*>(w_next + c);
      act_store4<AT>(out, (int64_t)t * width + c, make_float4((l.x - mean) * rstd * wv.x, (l.y - mean) * rstd * wv.y,
                                                                (l.z - mean) * rstd * wv.z, (l.w - mean) * rstd * wv.w));
    } else {
      act_store<AT>(out, (int64_t)t * width + c, (ln_row[c] - mean) * rstd * w_next[c]);
    }
  }
}

// ---------------------------------------------------------------------------------------
// What follows a fused q|k|v projection whose q and k are RMS-normalised over the WHOLE projection (all heads at once,
// with a weight), rotated over the leading rot_dims dimensions of each head in the interleaved layout (pair 2i, 2i+1;
// angles come from a cos|sin table that already carries any frequency scaling and magnitude factor), and whose values are
// brought to unit RMS per head and, when a value table is given, rotated over all their dimensions by their own
// position.  q leaves in fp32; k and v go to the paged cache (layout per layer [block][kv head][block_size][dim]).
// One CTA per token; everything fp32.  Tables: [pos][2][half] fp32 (cos row, then sin row).
// ---------------------------------------------------------------------------------------
template <typename AT, typename CT>
__global__ void __launch_bounds__(256)
qk_norm_rotate_cache_kernel(const AT* __restrict__ qkv, const float* __restrict__ qw, const float* __restrict__ kw,
                            const int32_t* __restrict__ positions, const int32_t* __restrict__ slots,
                            const float* __restrict__ rot, int rot_dims, const float* __restrict__ vrot,
                            float* __restrict__ qout, __nv_bfloat16* __restrict__ qout16, CT* kc, CT* vc, int heads, int kv_heads,
                            int dim, int vdim, int block_size, float eps, int64_t max_pos, int kstride, int vstride) {
  extern __shared__ float row[];
  __shared__ float red[8];
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int qn = heads * dim, kn = kv_heads * dim, vn = kv_heads * vdim, rw = qn + kn + vn;
  float* vr = row + rw;   // per kv head: 1 / rms of the value
  float sq = 0.f, sk = 0.f;
  const bool pairs = (vdim & 1) == 0;   // dim is even by contract: with an even vdim every row splits into aligned pairs
  if (pairs) {
    for (int c = threadIdx.x * 2; c < rw; c += blockDim.x * 2) {
      float v0, v1;
      if (sizeof(AT) == 4) {
        const float2 f = *reinterpret_cast<const float2*>(reinterpret_cast<const float*>(qkv) + (int64_t)t * rw + c);
        v0 = f.x;
        v1 = f.y;
      } else {
        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(reinterpret_cast<const __nv_bfloat16*>(qkv) + (int64_t)t * rw + c));
        v0 = f.x;
        v1 = f.y;
      }
      row[c] = v0;
      row[c + 1] = v1;
      if (c < qn) sq = fmaf(v1, v1, fmaf(v0, v0, sq));
      else if (c < qn + kn) sk = fmaf(v1, v1, fmaf(v0, v0, sk));
    }
  } else {
    for (int c = threadIdx.x; c < rw; c += blockDim.x) {
      const float v = act_load<AT>(qkv, (int64_t)t * rw + c);
      row[c] = v;
      if (c < qn) sq = fmaf(v, v, sq);
      else if (c < qn + kn) sk = fmaf(v, v, sk);
    }
  }
  const float rq = 1.0f / sqrtf(block_sum(sq, red) / (float)qn + eps);
  const float rk = 1.0f / sqrtf(block_sum(sk, red) / (float)kn + eps);
  {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int g = warp; g < kv_heads; g += blockDim.x >> 5) {
      float s = 0.f;
      for (int d = lane; d < vdim; d += 32) {
        const float v = row[qn + kn + g * vdim + d];
        s = fmaf(v, v, s);
      }
      s = warp_sum(s);
      if (lane == 0) vr[g] = 1.0f / sqrtf(s / (float)vdim + eps);
    }
  }
  __syncthreads();
  int pos = positions[t];
  pos = pos < 0 ? 0 : (pos >= max_pos ? (int)max_pos - 1 : pos);
  const int slot = slots[t];
  const int half = rot_dims >> 1, vhalf = vdim >> 1;
  const float* rc = rot ? rot + (int64_t)pos * rot_dims : nullptr;        // cos[half] | sin[half]
  const float* vcs = vrot ? vrot + (int64_t)pos * 2 * vhalf : nullptr;
  const int64_t blk = slot >= 0 ? slot / block_size : 0, off = slot >= 0 ? slot % block_size : 0;
  for (int c = threadIdx.x * 2; c < qn + kn; c += blockDim.x * 2) {   // pair (c, c + 1): dim and the bases are even
    const bool is_q = c < qn;
    const int e = is_q ? c : c - qn;
    const int d = e % dim;
    const float r = is_q ? rq : rk;
    const float* w = is_q ? qw : kw;
    float v0 = row[c] * r * w[e], v1 = row[c + 1] * r * w[e + 1];
    if (d < rot_dims && rc) {
      const int i = d >> 1;
      const float cs = rc[i], sn = rc[half + i];
      const float o0 = fmaf(v0, cs, -v1 * sn), o1 = fmaf(v1, cs, v0 * sn);
      v0 = o0;
      v1 = o1;
    }
    if (is_q) {
      // bf16 queries for the tensor-core attention kernels: heads as wide as the key cache's rows
      if (qout16) *reinterpret_cast<__nv_bfloat162*>(qout16 + ((int64_t)t * heads + e / dim) * kstride + d) = __floats2bfloat162_rn(v0, v1);
      else *reinterpret_cast<float2*>(qout + (int64_t)t * qn + e) = make_float2(v0, v1);
    } else if (slot >= 0) {
      const int g = e / dim;
      const int64_t at = ((blk * kv_heads + g) * block_size + off) * kstride + d;
      if (sizeof(CT) == 4) *reinterpret_cast<float2*>(reinterpret_cast<float*>(kc) + at) = make_float2(v0, v1);
      else *reinterpret_cast<__nv_bfloat162*>(reinterpret_cast<__nv_bfloat16*>(kc) + at) = __floats2bfloat162_rn(v0, v1);
    }
  }
  // rows wider than the head (a cache laid out for 128-wide kernels): the tail is kept at zero, so that it adds nothing
  // to a score and nothing to an output
  if (kstride > dim) {
    const int pad = kstride - dim;
    if (qout16)
      for (int c = threadIdx.x; c < heads * pad; c += blockDim.x)
        qout16[((int64_t)t * heads + c / pad) * kstride + dim + c % pad] = __float2bfloat16_rn(0.f);
    if (slot >= 0)
      for (int c = threadIdx.x; c < kv_heads * pad; c += blockDim.x) {
        const int64_t at = ((blk * kv_heads + c / pad) * block_size + off) * kstride + dim + c % pad;
        if (sizeof(CT) == 4) reinterpret_cast<float*>(kc)[at] = 0.f;
        else reinterpret_cast<__nv_bfloat16*>(kc)[at] = __float2bfloat16_rn(0.f);
      }
  }
  if (slot < 0) return;
  if (vstride > vdim) {
    const int pad = vstride - vdim;
    for (int c = threadIdx.x; c < kv_heads * pad; c += blockDim.x) {
      const int64_t at = ((blk * kv_heads + c / pad) * block_size + off) * vstride + vdim + c % pad;
      if (sizeof(CT) == 4) reinterpret_cast<float*>(vc)[at] = 0.f;
      else reinterpret_cast<__nv_bfloat16*>(vc)[at] = __float2bfloat16_rn(0.f);
    }
  }
  if (pairs) {
    for (int c = threadIdx.x * 2; c < vn; c += blockDim.x * 2) {
      const int g = c / vdim, d = c % vdim;
      float v0 = row[qn + kn + c] * vr[g], v1 = row[qn + kn + c + 1] * vr[g];
      if (vcs) {
        const int i = d >> 1;
        const float cs = vcs[i], sn = vcs[vhalf + i];
        const float o0 = fmaf(v0, cs, -v1 * sn), o1 = fmaf(v1, cs, v0 * sn);
        v0 = o0;
        v1 = o1;
      }
      const int64_t at = ((blk * kv_heads + g) * block_size + off) * vstride + d;
      if (sizeof(CT) == 4) *reinterpret_cast<float2*>(reinterpret_cast<float*>(vc) + at) = make_float2(v0, v1);
      else *reinterpret_cast<__nv_bfloat162*>(reinterpret_cast<__nv_bfloat16*>(vc) + at) = __floats2bfloat162_rn(v0, v1);
    }
    return;
  }
  for (int c = threadIdx.x; c < vn; c += blockDim.x) {
    const int g = c / vdim, d = c % vdim;
    float v = row[qn + kn + c] * vr[g];
    if (vcs && d < 2 * vhalf) {
      const int i = d >> 1;
      const float cs = vcs[i], sn = vcs[vhalf + i];
      const float o = row[qn + kn + (c ^ 1)] * vr[g];
      v = (d & 1) ? fmaf(v, cs, o * sn) : fmaf(v, cs, -o * sn);
    }
    if (sizeof(CT) == 4) reinterpret_cast<float*>(vc)[((blk * kv_heads + g) * block_size + off) * vstride + d] = v;
    else reinterpret_cast<__nv_bfloat16*>(vc)[((blk * kv_heads + g) * block_size + off) * vstride + d] = __float2bfloat16_rn(v);
  }
}

// Turns the rows of an attention output back by the query's position: pair (2m, 2m+1) of every head by -pos * f_m, from the
// table the cache writer used ([pos][cos half | sin half] fp32; null: no rotation).  The input heads may be wider than vdim
// (in_stride elements each, the output of kernels built for 128-wide heads); the output heads are packed.  bf16, one thread
// per pair; in == out is allowed when the widths agree.
__global__ void __launch_bounds__(256)
rotate_back_rows_kernel(const __nv_bfloat16* in, int in_stride, __nv_bfloat16* out, const int32_t* __restrict__ positions,
                        const float* __restrict__ vrot, int heads, int vdim, int64_t max_pos) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x, vhalf = vdim >> 1;
  int pos = positions[t];
  pos = pos < 0 ? 0 : (pos >= max_pos ? (int)max_pos - 1 : pos);
  const float* cs = vrot ? vrot + (int64_t)pos * 2 * vhalf : nullptr;
  const __nv_bfloat162* src = reinterpret_cast<const __nv_bfloat162*>(in + (int64_t)t * heads * in_stride);
  __nv_bfloat162* dst = reinterpret_cast<__nv_bfloat162*>(out + (int64_t)t * heads * vdim);
  for (int i = threadIdx.x; i < heads * vhalf; i += 256) {
    const int h = i / vhalf, m = i % vhalf;
    const float2 uv = __bfloat1622float2(src[h * (in_stride >> 1) + m]);
    const float c = cs ? cs[m] : 1.f, sn = cs ? cs[vhalf + m] : 0.f;
    dst[i] = __floats2bfloat162_rn(fmaf(uv.x, c, uv.y * sn), fmaf(uv.y, c, -uv.x * sn));
  }
}

// fp32 logits -> bf16 copy for the samplers
__global__ void __launch_bounds__(256)
f32_to_bf16_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out, int64_t n) {
  pdl_wait();
  pdl_launch_dependents();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    out[i] = __float2bfloat16_rn(in[i]);
}
__global__ void __launch_bounds__(256)
bf16_to_f32_kernel(const __nv_bfloat16* __restrict__ in, float* __restrict__ out, int64_t n) {
  pdl_wait();
  pdl_launch_dependents();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    out[i] = __bfloat162float(in[i]);
}
}  // namespace

int advance_rows(int32_t* ids, int32_t* positions, int32_t* slots, int32_t* ctx_lens, const int32_t* block_table,
                 int bt_stride, const int32_t* row_to_seq, const int32_t* sampled, int n, int block_size,
                 cudaStream_t s) {
  if (n == 0) return B200_OK;
  B200_CUDA(launch(advance_rows_kernel, dim3((n + 127) / 128), dim3(128), 0, s, ids, positions, slots, ctx_lens,
                   block_table, bt_stride, row_to_seq, sampled, n, block_size));
  return B200_OK;
}

int embed(const int32_t* ids, const __nv_bfloat16* table, __nv_bfloat16* out, int T, int hidden, int vocab,
          cudaStream_t s, const int32_t* prev, int n_prev) {
  B200_REQUIRE(hidden % 8 == 0, B200_ERR_UNSUPPORTED, "embed: hidden %% 8 != 0");
  if (T == 0) return B200_OK;
  B200_CUDA(launch(embed_kernel, dim3(T), dim3(128), 0, s, ids, table, out, hidden, vocab, prev, n_prev));
  return B200_OK;
}

int rmsnorm(const __nv_bfloat16* x, __nv_bfloat16* res, const __nv_bfloat16* w, __nv_bfloat16* y, int T,
            int hidden, float eps, cudaStream_t s) {
  B200_REQUIRE(hidden % 128 == 0 && hidden <= 128 * kNormWarps * kNormMaxSlabs, B200_ERR_UNSUPPORTED,
               "rmsnorm: hidden=%d unsupported (multiple of 128, <= %d)", hidden, 128 * kNormWarps * kNormMaxSlabs);
  if (T == 0) return B200_OK;
  if (res)
    B200_CUDA(launch(rmsnorm_kernel<true>, dim3(T), dim3(kNormThreads), 0, s, x, res, w, y, hidden, eps));
  else
    B200_CUDA(launch(rmsnorm_kernel<false>, dim3(T), dim3(kNormThreads), 0, s, x, res, w, y, hidden, eps));
  return B200_OK;
}

int embed_stream(const int32_t* ids, const __nv_bfloat16* table, float* sres, float* ssq, int T, int hidden, int vocab,
                 cudaStream_t s, const int32_t* prev, int n_prev) {
  B200_REQUIRE(hidden % 128 == 0, B200_ERR_UNSUPPORTED, "embed_stream: hidden %% 128 != 0");
  if (T == 0) return B200_OK;
  B200_CUDA(launch(embed_stream_kernel, dim3(T), dim3(kNormThreads), 0, s, ids, table, sres, ssq, hidden, vocab, prev, n_prev));
  return B200_OK;
}

int rmsnorm_stream(const float* sres, const float* ssq, const int32_t* rows, const __nv_bfloat16* w, __nv_bfloat16* y,
                   int R, int hidden, float eps, cudaStream_t s) {
  B200_REQUIRE(hidden % 128 == 0, B200_ERR_UNSUPPORTED, "rmsnorm_stream: hidden %% 128 != 0");
  if (R == 0) return B200_OK;
  B200_CUDA(launch(rmsnorm_stream_kernel, dim3(R), dim3(kNormThreads), 0, s, sres, ssq, rows, w, y, hidden, eps));
  return B200_OK;
}

int embed_scaled(const int32_t* ids, const __nv_bfloat16* table, float* out, int T, int width, int vocab, float scale,
                 cudaStream_t s, const int32_t* prev, int n_prev) {
  if (T == 0) return B200_OK;
  B200_CUDA(launch(embed_scaled_kernel, dim3(T), dim3(128), 0, s, ids, table, out, width, vocab, scale, prev, n_prev));
  return B200_OK;
}

template <typename AT>
static int layernorm_stream_t(float* x, const void* y, const float* yparts, int n_parts, const float* w_post,
                              const float* w_next, void* out, const int32_t* rows, int T, int width, float eps, cudaStream_t s) {
  if (T == 0) return B200_OK;
  const size_t smem = (size_t)width * 4;
  B200_REQUIRE(smem <= 200 * 1024, B200_ERR_UNSUPPORTED, "layernorm: width %d too large", width);
  const uintptr_t ptrs = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(yparts) |
                         reinterpret_cast<uintptr_t>(w_post) | reinterpret_cast<uintptr_t>(w_next) | reinterpret_cast<uintptr_t>(out);
  if (width % 4 == 0 && ptrs % 16 == 0) {
    static bool done4[64] = {};
    if (smem > 48 * 1024) B200_CUDA(ensure_dynamic_smem(layernorm_stream_kernel<AT, 4>, 200 * 1024, done4));
    B200_CUDA(launch(layernorm_stream_kernel<AT, 4>, dim3(T), dim3(kLnThreads), smem, s, x, (const AT*)y, yparts, n_parts, w_post,
                     w_next, (AT*)out, rows, width, eps));
    return B200_OK;
  }
  static bool done[64] = {};
  if (smem > 48 * 1024) B200_CUDA(ensure_dynamic_smem(layernorm_stream_kernel<AT, 1>, 200 * 1024, done));
  B200_CUDA(launch(layernorm_stream_kernel<AT, 1>, dim3(T), dim3(kLnThreads), smem, s, x, (const AT*)y, yparts, n_parts, w_post,
                   w_next, (AT*)out, rows, width, eps));
  return B200_OK;
}
int layernorm_stream(bool f32, float* x, const void* y, const float* yparts, int n_parts, const float* w_post,
                     const float* w_next, void* out, const int32_t* rows, int T, int width, float eps, cudaStream_t s) {
  B200_REQUIRE(!(y || yparts) || w_post, B200_ERR_INVALID, "layernorm: a sublayer output needs its norm weight");
  B200_REQUIRE(!w_next || out, B200_ERR_INVALID, "layernorm: no output for the normed rows");
  return f32 ? layernorm_stream_t<float>(x, y, yparts, n_parts, w_post, w_next, out, rows, T, width, eps, s)
             : layernorm_stream_t<__nv_bfloat16>(x, y, yparts, n_parts, w_post, w_next, out, rows, T, width, eps, s);
}

int qk_norm_rotate_cache(bool f32, const void* qkv, const float* qw, const float* kw, const int32_t* positions,
                         const int32_t* slots, const float* rot, int rot_dims, const float* vrot, float* qout, void* kc,
                         void* vc, int T, int heads, int kv_heads, int dim, int vdim, int block_size, float eps,
                         int64_t max_pos, cudaStream_t s, __nv_bfloat16* qout16, int kstride, int vstride) {
  if (T == 0) return B200_OK;
  if (kstride <= 0) kstride = dim;
  if (vstride <= 0) vstride = vdim;
  B200_REQUIRE(kstride >= dim && vstride >= vdim, B200_ERR_INVALID, "rotation: cache rows narrower than the heads");
  B200_REQUIRE(!(f32 && qout16), B200_ERR_INVALID, "rotation: bf16 queries are for the bf16 mode");
  B200_REQUIRE(dim % 2 == 0 && rot_dims % 2 == 0 && rot_dims <= dim && (vrot == nullptr || vdim % 2 == 0), B200_ERR_UNSUPPORTED,
               "rotation: head sizes must be even (dim %d, rot_dims %d, vdim %d)", dim, rot_dims, vdim);
  const size_t smem = ((size_t)heads * dim + (size_t)kv_heads * (dim + vdim) + kv_heads) * 4;
  B200_REQUIRE(smem <= 200 * 1024, B200_ERR_UNSUPPORTED, "qkv row of %zu bytes does not fit shared memory", smem);
  static bool done[2][64] = {};
  if (f32) {
    if (smem > 48 * 1024) B200_CUDA(ensure_dynamic_smem(qk_norm_rotate_cache_kernel<float, float>, 200 * 1024, done[0]));
    B200_CUDA(launch(qk_norm_rotate_cache_kernel<float, float>, dim3(T), dim3(256), smem, s, (const float*)qkv, qw, kw, positions,
                     slots, rot, rot_dims, vrot, qout, (__nv_bfloat16*)nullptr, (float*)kc, (float*)vc, heads, kv_heads, dim, vdim, block_size, eps, max_pos, kstride, vstride));
  } else {
    if (smem > 48 * 1024)
      B200_CUDA(ensure_dynamic_smem(qk_norm_rotate_cache_kernel<__nv_bfloat16, __nv_bfloat16>, 200 * 1024, done[1]));
    B200_CUDA(launch(qk_norm_rotate_cache_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(T), dim3(256), smem, s,
                     (const __nv_bfloat16*)qkv, qw, kw, positions, slots, rot, rot_dims, vrot, qout, qout16, (__nv_bfloat16*)kc,
                     (__nv_bfloat16*)vc, heads, kv_heads, dim, vdim, block_size, eps, max_pos, kstride, vstride));
  }
  return B200_OK;
}

int rotate_back_rows(const __nv_bfloat16* in, int in_stride, __nv_bfloat16* out, const int32_t* positions, const float* vrot, int T,
                     int heads, int vdim, int64_t max_pos, cudaStream_t s) {
  B200_REQUIRE(vdim % 2 == 0 && in_stride % 2 == 0 && in_stride >= vdim &&
                   ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 3) == 0 && (in != out || in_stride == vdim),
               B200_ERR_UNSUPPORTED, "rotate_back: vdim %d in rows of %d", vdim, in_stride);
  if (T == 0) return B200_OK;
  B200_CUDA(launch(rotate_back_rows_kernel, dim3(T), dim3(256), (size_t)0, s, in, in_stride, out, positions, vrot, heads, vdim, max_pos));
  return B200_OK;
}

int convert_f32_to_bf16(const float* in, __nv_bfloat16* out, int64_t n, cudaStream_t s) {
  if (n == 0) return B200_OK;
  const int grid = (int)std::min<int64_t>((n + 255) / 256, (int64_t)kNumSMs * 8);
  B200_CUDA(launch(f32_to_bf16_kernel, dim3(grid), dim3(256), 0, s, in, out, n));
  return B200_OK;
}
int convert_bf16_to_f32(const __nv_bfloat16* in, float* out, int64_t n, cudaStream_t s) {
  if (n == 0) return B200_OK;
  const int grid = (int)std::min<int64_t>((n + 255) / 256, (int64_t)kNumSMs * 8);
  B200_CUDA(launch(bf16_to_f32_kernel, dim3(grid), dim3(256), 0, s, in, out, n));
  return B200_OK;
}

int rope_kv_append(__nv_bfloat16* qkv, const int32_t* positions, const int32_t* slots,
                   const __nv_bfloat16* cos_sin, __nv_bfloat16* kc, __nv_bfloat16* vc, int T, int hq,
                   int hkv, int block_size, cudaStream_t s) {
  if (T == 0) return B200_OK;
  B200_CUDA(launch(rope_kv_kernel, dim3(T, hq + 2 * hkv), dim3(64), 0, s, qkv, positions, slots, cos_sin, kc, vc,
                   hq, hkv, block_size));
  return B200_OK;
}

int silu_mul(const __nv_bfloat16* gu, __nv_bfloat16* out, int T, int inter, cudaStream_t s) {
  B200_REQUIRE(inter % 8 == 0, B200_ERR_UNSUPPORTED, "silu_mul: intermediate %% 8 != 0");
  if (T == 0) return B200_OK;
  const int64_t chunks = (int64_t)T * (inter / 8);
  int64_t grid64 = (chunks + 255) / 256;
  if (grid64 > (int64_t)kNumSMs * 8) grid64 = (int64_t)kNumSMs * 8;
  const int grid = (int)grid64;
  B200_CUDA(launch(silu_mul_kernel, dim3(grid), dim3(256), 0, s, gu, out, inter, chunks));
  return B200_OK;
}

int argmax_rows(const __nv_bfloat16* logits, int64_t ld, int rows, int vocab, int index_offset,
                int32_t* out_ids, float* out_max, cudaStream_t s) {
  B200_REQUIRE(ld % 8 == 0, B200_ERR_UNSUPPORTED, "argmax: ld %% 8 != 0");
  if (rows == 0) return B200_OK;
  B200_CUDA(launch(argmax_kernel, dim3(rows), dim3(kArgmaxThreads), 0, s, logits, ld, vocab, index_offset, out_ids,
                   out_max));
  return B200_OK;
}

}  // namespace b200
