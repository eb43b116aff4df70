// Matrix-memory recurrence (B200_MIXER_MLSTM).  Per head and sequence the state is S [dim][vdim], n [dim] and a running
// maximum m of the log gates, all fp32, kept in the sequence's state slot between steps:
//   i_t = cap tanh((w_i . h + b_i) / cap)              f_t = logsigmoid(cap tanh((w_f . h + b_f) / cap))
//   m_t = max(f_t + m_{t-1}, i_t)                      a = exp(f_t + m_{t-1} - m_t),  b = exp(i_t - m_t)
//   S_t = a S_{t-1} + b k_t v_t^T                      n_t = a n_{t-1} + b k_t
//   o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6),   q_t scaled by dim^-1/2
// then each head's o_t is brought to unit RMS, multiplied by a weight and by sigmoid(g_t).
//
//  * mlstm_gates: the two gate projections with fp32 accumulation and the gate transforms, [T][2 heads] fp32;
//  * mlstm_scan: the recurrence.  One CTA per (sequence, head, 32 value columns) walks the sequence's rows of the step in
//    order (a decode row is a walk of one), 16 rows staged in shared memory at a time; a warp owns 4 columns, a lane the
//    key dimensions lane, lane + 32, ...; the state lives in registers during the walk and is stored as [head][vdim][dim] so that a warp's loads are contiguous.
//    n and m are kept once per CTA (every CTA of a head needs them from the step before, so they cannot share one copy
//    that one of them overwrites).  A sequence whose first row is at position 0 starts from zeros.
//  * head_norm_gate: unit RMS per head, weight, sigmoid gate.
#include "common.cuh"

namespace b200 {
namespace {

template <typename AT> __device__ __forceinline__ float ldx(const AT* p, int64_t i);
template <> __device__ __forceinline__ float ldx<float>(const float* p, int64_t i) { return p[i]; }
template <> __device__ __forceinline__ float ldx<__nv_bfloat16>(const __nv_bfloat16* p, int64_t i) { return __bfloat162float(p[i]); }
template <typename AT> __device__ __forceinline__ void stx(AT* p, int64_t i, float v);
template <> __device__ __forceinline__ void stx<float>(float* p, int64_t i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void stx<__nv_bfloat16>(__nv_bfloat16* p, int64_t i, float v) { p[i] = __float2bfloat16_rn(v); }

__device__ __forceinline__ float log_sigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

template <typename AT>
__global__ void __launch_bounds__(128)
mlstm_gates_kernel(const AT* __restrict__ x, const __nv_bfloat16* __restrict__ w, const float* __restrict__ bias, float* __restrict__ out,
                   int width, int heads, float cap) {
  extern __shared__ float xs[];
  pdl_wait();
  pdl_launch_dependents();
  const int64_t t = blockIdx.x;
  for (int c = threadIdx.x; c < width; c += 128) xs[c] = ldx<AT>(x, t * width + c);
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int o = warp; o < 2 * heads; o += 4) {
    const __nv_bfloat16* wr = w + (int64_t)o * width;
    float a = 0.f;
    for (int c = lane; c < width; c += 32) a = fmaf(__bfloat162float(wr[c]), xs[c], a);
    a = warp_sum(a);
    if (lane == 0) {
      const float z = cap * tanhf((a + (bias ? bias[o] : 0.f)) / cap);
      out[t * 2 * heads + o] = o < heads ? z : log_sigmoid(z);
    }
  }
}

constexpr int kScanCols = 4;                 // value columns per warp
constexpr int kScanWarps = 8;
constexpr int kScanBlockCols = kScanCols * kScanWarps;
constexpr int kScanStage = 16;               // rows staged in shared memory at a time

template <typename AT, int DPL>
__global__ void __launch_bounds__(kScanWarps * 32)
mlstm_scan_kernel(const AT* __restrict__ qkv, int64_t ld, int q_off, int k_off, int v_off, const float* __restrict__ gates,
                  const int32_t* __restrict__ positions, const int32_t* __restrict__ seq_start, const int32_t* __restrict__ seq_slots,
                  float* __restrict__ state, int64_t slot_stride, float* __restrict__ out, int heads, int dim, int vd, float qscale) {
  pdl_wait();
  pdl_launch_dependents();
  const int s = blockIdx.x, h = blockIdx.y, zb = blockIdx.z, nz = gridDim.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int start = seq_start[s], n_rows = seq_start[s + 1] - start;
  if (n_rows <= 0) return;
  const bool fresh = positions[start] == 0;
  float* S_st = state + (int64_t)seq_slots[s] * slot_stride;                  // [heads][vd][dim]
  float* n_st = S_st + (int64_t)heads * vd * dim + ((int64_t)h * nz + zb) * dim;   // [heads][nz][dim]
  float* m_st = S_st + (int64_t)heads * vd * dim + (int64_t)heads * nz * dim + (int64_t)h * nz + zb;   // [heads][nz]
  const int j0 = zb * kScanBlockCols + warp * kScanCols;
  float Sr[kScanCols][DPL], nr[DPL];
#pragma unroll
  for (int i = 0; i < DPL; ++i) {
    const int d = lane + 32 * i;
    nr[i] = (!fresh && d < dim) ? n_st[d] : 0.f;
#pragma unroll
    for (int c = 0; c < kScanCols; ++c)
      Sr[c][i] = (!fresh && d < dim && j0 + c < vd) ? S_st[((int64_t)h * vd + j0 + c) * dim + d] : 0.f;
  }
  float m = fresh ? 0.f : *m_st;
  __syncthreads();   // every warp has read n and m before warp 0 may store them
  // The rows of the step are staged kScanStage at a time: q (scaled), k, this CTA's 32 value columns and the two gates of
  // the head, loaded by the whole CTA with one round trip to memory per stage; the walk itself reads shared memory only.
  extern __shared__ float stage[];
  float* sq = stage;                          // [kScanStage][dim]
  float* sk = sq + kScanStage * dim;          // [kScanStage][dim]
  float* sv = sk + kScanStage * dim;          // [kScanStage][32]
  float* sg = sv + kScanStage * kScanBlockCols;   // [kScanStage][2]
  const int jb = zb * kScanBlockCols;
  for (int b0 = 0; b0 < n_rows; b0 += kScanStage) {
    const int nb = min(kScanStage, n_rows - b0);
    __syncthreads();   // the stage before has been consumed
    for (int e = threadIdx.x; e < nb * dim; e += kScanWarps * 32) {
      const int r = e / dim, d = e % dim;
      const AT* row = qkv + (int64_t)(start + b0 + r) * ld;
      sq[e] = ldx<AT>(row, q_off + h * dim + d) * qscale;
      sk[e] = ldx<AT>(row, k_off + h * dim + d);
    }
    for (int e = threadIdx.x; e < nb * kScanBlockCols; e += kScanWarps * 32) {
      const int r = e / kScanBlockCols, j = jb + e % kScanBlockCols;
      sv[e] = j < vd ? ldx<AT>(qkv + (int64_t)(start + b0 + r) * ld, v_off + h * vd + j) : 0.f;
    }
    for (int e = threadIdx.x; e < nb * 2; e += kScanWarps * 32)
      sg[e] = gates[(int64_t)(start + b0 + (e >> 1)) * 2 * heads + (e & 1) * heads + h];
    __syncthreads();
    for (int r = 0; r < nb; ++r) {
      const int t = start + b0 + r;
      float q[DPL], k[DPL], v[kScanCols];
      const float ig = sg[2 * r], fg = sg[2 * r + 1];
#pragma unroll
      for (int i = 0; i < DPL; ++i) {
        const int d = lane + 32 * i;
        q[i] = d < dim ? sq[r * dim + d] : 0.f;
        k[i] = d < dim ? sk[r * dim + d] : 0.f;
      }
#pragma unroll
      for (int c = 0; c < kScanCols; ++c) v[c] = sv[r * kScanBlockCols + warp * kScanCols + c];
      const float m_new = fmaxf(fg + m, ig);
      const float a = expf(fg + m - m_new), b = expf(ig - m_new);
      m = m_new;
      float nq = 0.f, acc[kScanCols];
#pragma unroll
      for (int c = 0; c < kScanCols; ++c) acc[c] = 0.f;
#pragma unroll
      for (int i = 0; i < DPL; ++i) {
        const float bk = b * k[i];
        nr[i] = fmaf(a, nr[i], bk);
        nq = fmaf(nr[i], q[i], nq);
#pragma unroll
        for (int c = 0; c < kScanCols; ++c) {
          Sr[c][i] = fmaf(a, Sr[c][i], bk * v[c]);
          acc[c] = fmaf(Sr[c][i], q[i], acc[c]);
        }
      }
      nq = warp_sum(nq);
      const float den = fmaxf(fabsf(nq), expf(-m)) + 1e-6f;
      float mine = 0.f;
#pragma unroll
      for (int c = 0; c < kScanCols; ++c) {
        const float o = warp_sum(acc[c]);
        if (lane == c) mine = o;
      }
      if (lane < kScanCols && j0 + lane < vd) out[((int64_t)t * heads + h) * vd + j0 + lane] = mine / den;
    }
  }
#pragma unroll
  for (int i = 0; i < DPL; ++i) {
    const int d = lane + 32 * i;
    if (d < dim) {
      if (warp == 0) n_st[d] = nr[i];
#pragma unroll
      for (int c = 0; c < kScanCols; ++c)
        if (j0 + c < vd) S_st[((int64_t)h * vd + j0 + c) * dim + d] = Sr[c][i];
    }
  }
  if (warp == 0 && lane == 0) *m_st = m;
}

// one CTA per row, one warp per head (round robin)
template <typename AT>
__global__ void __launch_bounds__(128)
head_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ w, const AT* __restrict__ gate, int64_t ldg,
                      AT* __restrict__ out, int heads, int vd, float eps) {
  pdl_wait();
  pdl_launch_dependents();
  const int64_t t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int h = warp; h < heads; h += 4) {
    const float* src = o + (t * heads + h) * vd;
    float ss = 0.f;
    for (int j = lane; j < vd; j += 32) ss = fmaf(src[j], src[j], ss);
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)vd + eps);
    for (int j = lane; j < vd; j += 32) {
      float v = src[j] * inv;
      if (w) v *= w[h * vd + j];
      if (gate) v *= 1.0f / (1.0f + expf(-ldx<AT>(gate, t * ldg + h * vd + j)));
      stx<AT>(out, (t * heads + h) * vd + j, v);
    }
  }
}

}  // namespace

int mlstm_gates(bool f32, const void* x, const __nv_bfloat16* w, const float* bias, float* out, int T, int width, int heads, float cap,
                cudaStream_t s) {
  if (T == 0) return B200_OK;
  B200_REQUIRE(cap > 0.f, B200_ERR_INVALID, "mlstm_gates: cap %f", (double)cap);
  const size_t smem = (size_t)width * 4;
  B200_REQUIRE(smem <= 200 * 1024, B200_ERR_UNSUPPORTED, "mlstm_gates: width %d does not fit shared memory", width);
  static bool done[2][64] = {};
  if (f32) {
    if (smem > 48 * 1024) B200_CUDA(ensure_dynamic_smem(mlstm_gates_kernel<float>, 200 * 1024, done[0]));
    B200_CUDA(launch(mlstm_gates_kernel<float>, dim3(T), dim3(128), smem, s, (const float*)x, w, bias, out, width, heads, cap));
  } else {
    if (smem > 48 * 1024) B200_CUDA(ensure_dynamic_smem(mlstm_gates_kernel<__nv_bfloat16>, 200 * 1024, done[1]));
    B200_CUDA(launch(mlstm_gates_kernel<__nv_bfloat16>, dim3(T), dim3(128), smem, s, (const __nv_bfloat16*)x, w, bias, out, width, heads,
                     cap));
  }
  return B200_OK;
}

int mlstm_col_blocks(int vd) { return (vd + kScanBlockCols - 1) / kScanBlockCols; }

// floats of one layer's recurrent state in a slot: S [heads][vd][dim], n [heads][col blocks][dim], m [heads][col blocks]
int64_t mlstm_state_floats(int heads, int dim, int vd) {
  const int64_t nz = mlstm_col_blocks(vd);
  return (int64_t)heads * vd * dim + (int64_t)heads * nz * dim + (int64_t)heads * nz;
}

template <typename AT>
static int mlstm_scan_t(const void* qkv, int64_t ld, int q_off, int k_off, int v_off, const float* gates, const int32_t* positions,
                        const int32_t* seq_start, const int32_t* seq_slots, float* state, int64_t slot_stride, float* out, int S,
                        int heads, int dim, int vd, cudaStream_t s) {
  const dim3 grid(S, heads, mlstm_col_blocks(vd)), block(kScanWarps * 32);
  const float qscale = 1.0f / sqrtf((float)dim);
  const int dpl = (dim + 31) / 32;
  const size_t smem = (size_t)kScanStage * (2 * dim + kScanBlockCols + 2) * 4;   // <= 34 KiB for dim <= 256
#define SCAN(D)                                                                                                                   \
  B200_CUDA(launch(mlstm_scan_kernel<AT, D>, grid, block, smem, s, (const AT*)qkv, ld, q_off, k_off, v_off, gates, positions, \
                   seq_start, seq_slots, state, slot_stride, out, heads, dim, vd, qscale))
  if (dpl <= 1) SCAN(1);
  else if (dpl <= 2) SCAN(2);
  else if (dpl <= 4) SCAN(4);
  else SCAN(8);
#undef SCAN
  return B200_OK;
}

int mlstm_scan(bool f32, const void* qkv, int64_t ld, int q_off, int k_off, int v_off, const float* gates, const int32_t* positions,
               const int32_t* seq_start, const int32_t* seq_slots, float* state, int64_t slot_stride, float* out, int S, int heads,
               int dim, int vd, cudaStream_t s) {
  if (S == 0) return B200_OK;
  B200_REQUIRE(dim > 0 && dim <= 256 && vd > 0, B200_ERR_UNSUPPORTED, "mlstm_scan: key size %d outside (0, 256]", dim);
  B200_REQUIRE(positions && seq_start && seq_slots && state, B200_ERR_INVALID, "mlstm_scan: null argument");
  return f32 ? mlstm_scan_t<float>(qkv, ld, q_off, k_off, v_off, gates, positions, seq_start, seq_slots, state, slot_stride, out, S, heads,
                                   dim, vd, s)
             : mlstm_scan_t<__nv_bfloat16>(qkv, ld, q_off, k_off, v_off, gates, positions, seq_start, seq_slots, state, slot_stride, out,
                                           S, heads, dim, vd, s);
}

int head_norm_gate(bool f32, const float* o, const float* w, const void* gate, int64_t ldg, void* out, int T, int heads, int vd, float eps,
                   cudaStream_t s) {
  if (T == 0) return B200_OK;
  if (f32)
    B200_CUDA(launch(head_norm_gate_kernel<float>, dim3(T), dim3(128), (size_t)0, s, o, w, (const float*)gate, ldg, (float*)out, heads, vd,
                     eps));
  else
    B200_CUDA(launch(head_norm_gate_kernel<__nv_bfloat16>, dim3(T), dim3(128), (size_t)0, s, o, w, (const __nv_bfloat16*)gate, ldg,
                     (__nv_bfloat16*)out, heads, vd, eps));
  return B200_OK;
}

}  // namespace b200
