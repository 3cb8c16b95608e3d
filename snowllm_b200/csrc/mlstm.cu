// Matrix memory with exponential gates (mLSTM), token by token, over a flat batch of segments.
//
// Per head: a matrix S [dk, dv], a vector n [dk] and a running maximum m, all float, all zero for a
// fresh request (m too), kept in the request's state slot between steps.  With i_t and f_t the log
// input and log forget gates of the token:
//
//   i = cap * tanh((x_i + b_i) / cap),  f = logsigmoid(cap * tanh((x_f + b_f) / cap))
//   m' = max(f + m, i);  S' = exp(f + m - m') S + exp(i - m') k v^T;  n' likewise with k alone
//   o = S'^T q / (max(|n' . q|, exp(-m')) + 1e-6),   q scaled by dk^(-1/2)
//
// A block serves one (segment, head, 32 columns of S).  Eight neighbouring threads share a column: each
// holds an eighth of its rows in registers over the whole segment (rows in groups of four, dealt round
// robin, so that the eight read one contiguous piece of k and q), and three shuffles add their parts of
// S^T q.  n is kept by every warp for itself, so the warps never wait for one another inside a chunk: the
// block meets only to bring the next 32 tokens' q, k, v into shared memory and to work out their gates:
// the running maximum is a short serial scan by one thread, the three exponentials per token (keep, take,
// exp(-m)) are then taken by one thread per token, off the token loop's chain of dependent instructions.  The output is the raw o in float; the per-head norm, the weight and the
// output gate follow in head_norm_gate (sublayer.cu).  Everything here is 32-bit.
#include "common.cuh"

#define ML_CHUNK 32

__device__ __forceinline__ float log_sigmoid_f(float z) {
  return fminf(z, 0.f) - log1pf(expf(-fabsf(z)));
}

#define ML_COLS 32             // columns of S per block
#define ML_TPC 8               // threads per column

template <int DKR>
__global__ void __launch_bounds__(ML_TPC * ML_COLS)
mlstm_kernel(const float* __restrict__ proj, long long ld, int q_off, int k_off, int v_off,
             int i_off, int f_off, SmallVec bias_i, SmallVec bias_f, float cap,
             const int* __restrict__ cu_seqlens, const int* __restrict__ seg_start,
             const int* __restrict__ seg_slot, float* __restrict__ state_s,
             float* __restrict__ state_n, float* __restrict__ state_m,
             float* __restrict__ out, int H, int dk, int dv) {
  pdl_begin();
  extern __shared__ __align__(16) float ml_sh[];
  constexpr int RPT = DKR / ML_TPC;                      // rows of S per thread
  const int b = blockIdx.x, h = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = threadIdx.x & (ML_TPC - 1);            // which share of the column's rows
  const int c = blockIdx.z * ML_COLS + threadIdx.x / ML_TPC;
  const bool has_col = c < dv;
  const int dkp = (dk + 4 * ML_TPC - 1) / (4 * ML_TPC) * (4 * ML_TPC);
  float* qs = ml_sh;                                     // [ML_CHUNK][dkp]
  float* ks = qs + ML_CHUNK * dkp;                       // [ML_CHUNK][dkp]
  float* vs = ks + ML_CHUNK * dkp;                       // [ML_CHUNK][ML_COLS]
  float* gi = vs + ML_CHUNK * ML_COLS;                   // [ML_CHUNK]
  float* gf = gi + ML_CHUNK;                             // [ML_CHUNK]
  float* g_keep = gf + ML_CHUNK;                         // exp(f + m' - m), exp(i - m), exp(-m), m and m' per token
  float* g_take = g_keep + ML_CHUNK;
  float* g_en = g_take + ML_CHUNK;
  float* g_m = g_en + ML_CHUNK;
  float* g_mprev = g_m + ML_CHUNK;

  const int row0 = cu_seqlens[b], row1 = cu_seqlens[b + 1];
  const int slot = seg_slot[b];
  const bool fresh = seg_start[b] == 0;
  float* Ss = state_s + ((size_t)slot * H + h) * dk * dv;
  float* Sn = state_n + ((size_t)slot * H + h) * dk;
  float* Sm = state_m + (size_t)slot * H + h;

  // register i*4 + e holds row 4 ML_TPC i + 4 sub + e
  float S[RPT], n[DKR / 32];
  float m = 0.f;
#pragma unroll
  for (int i = 0; i < RPT / 4; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int r = 4 * ML_TPC * i + 4 * sub + e;
      S[i * 4 + e] = (!fresh && has_col && r < dk) ? Ss[(size_t)r * dv + c] : 0.f;
    }
#pragma unroll
  for (int j = 0; j < DKR / 32; ++j) n[j] = (!fresh && lane + 32 * j < dk) ? Sn[lane + 32 * j] : 0.f;
  if (!fresh) m = *Sm;
  const float q_scale = 1.f / sqrtf((float)dk);
  const float inv_cap = 1.f / cap;
  const float bi = bias_i[h], bf = bias_f[h];
  const int col0 = blockIdx.z * ML_COLS;

  for (int t0 = row0; t0 < row1; t0 += ML_CHUNK) {
    const int nt = min(ML_CHUNK, row1 - t0);
    __syncthreads();                                     // everyone is done with the previous chunk
    for (int i = threadIdx.x; i < nt * dkp; i += blockDim.x) {
      const int t = i / dkp, r = i - t * dkp;
      const float* pr = proj + (size_t)(t0 + t) * ld;
      qs[i] = r < dk ? pr[q_off + h * dk + r] * q_scale : 0.f;
      ks[i] = r < dk ? pr[k_off + h * dk + r] : 0.f;
    }
    for (int i = threadIdx.x; i < nt * ML_COLS; i += blockDim.x) {
      const int t = i / ML_COLS, d = i - t * ML_COLS;
      vs[i] = col0 + d < dv ? proj[(size_t)(t0 + t) * ld + v_off + h * dv + col0 + d] : 0.f;
    }
    for (int t = threadIdx.x; t < nt; t += blockDim.x) {
      const float* pr = proj + (size_t)(t0 + t) * ld;
      gi[t] = cap * tanhf((pr[i_off + h] + bi) * inv_cap);
      gf[t] = log_sigmoid_f(cap * tanhf((pr[f_off + h] + bf) * inv_cap));
    }
    __syncthreads();
    if (threadIdx.x == 0) {                              // the running maximum: a serial scan of two operations a token
      float mm = m;
      for (int t = 0; t < nt; ++t) {
        g_mprev[t] = mm;
        mm = fmaxf(gf[t] + mm, gi[t]);
        g_m[t] = mm;
      }
    }
    __syncthreads();
    if (threadIdx.x < nt) {
      const int t = threadIdx.x;
      g_keep[t] = expf(gf[t] + g_mprev[t] - g_m[t]);
      g_take[t] = expf(gi[t] - g_m[t]);
      g_en[t] = expf(-g_m[t]);
    }
    __syncthreads();
    m = g_m[nt - 1];
    // Only S and n pass from one token to the next (one multiply-add each); the sums, shuffles and the division of
    // neighbouring tokens are independent, so four tokens' worth of them are kept in flight.
#pragma unroll 4
    for (int t = 0; t < nt; ++t) {
      const float keep = g_keep[t], take = g_take[t];
      const float* qt = qs + t * dkp;
      const float* kt = ks + t * dkp;
      const float tv = take * vs[t * ML_COLS + threadIdx.x / ML_TPC];
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < RPT / 4; ++i) {
        if (4 * ML_TPC * i < dk) {
          const float4 k4 = *reinterpret_cast<const float4*>(kt + 4 * ML_TPC * i + 4 * sub);
          const float4 q4 = *reinterpret_cast<const float4*>(qt + 4 * ML_TPC * i + 4 * sub);
          S[i * 4 + 0] = fmaf(keep, S[i * 4 + 0], k4.x * tv); acc = fmaf(S[i * 4 + 0], q4.x, acc);
          S[i * 4 + 1] = fmaf(keep, S[i * 4 + 1], k4.y * tv); acc = fmaf(S[i * 4 + 1], q4.y, acc);
          S[i * 4 + 2] = fmaf(keep, S[i * 4 + 2], k4.z * tv); acc = fmaf(S[i * 4 + 2], q4.z, acc);
          S[i * 4 + 3] = fmaf(keep, S[i * 4 + 3], k4.w * tv); acc = fmaf(S[i * 4 + 3], q4.w, acc);
        }
      }
#pragma unroll
      for (int w = 1; w < ML_TPC; w <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, w);
      float dot = 0.f;
#pragma unroll
      for (int j = 0; j < DKR / 32; ++j) {
        const int r = lane + 32 * j;
        if (r < dk) {
          n[j] = fmaf(keep, n[j], take * kt[r]);
          dot = fmaf(n[j], qt[r], dot);
        }
      }
      dot = warp_sum(dot);
      const float below = fmaxf(fabsf(dot), g_en[t]) + 1e-6f;
      if (has_col && sub == 0) out[(size_t)(t0 + t) * H * dv + (size_t)h * dv + c] = acc / below;
    }
  }
#pragma unroll
  for (int i = 0; i < RPT / 4; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int r = 4 * ML_TPC * i + 4 * sub + e;
      if (has_col && r < dk) Ss[(size_t)r * dv + c] = S[i * 4 + e];
    }
  if (warp == 0 && blockIdx.z == 0) {
#pragma unroll
    for (int j = 0; j < DKR / 32; ++j)
      if (lane + 32 * j < dk) Sn[lane + 32 * j] = n[j];
    if (lane == 0) *Sm = m;
  }
}

// proj: float [M, ld] with q ([H, dk]) at q_off, k at k_off, v ([H, dv]) at v_off and the two gates'
// pre-activations ([H] each) at i_off and f_off.  state_s [slots, H, dk, dv], state_n [slots, H, dk],
// state_m [slots, H].  out: float [M, H*dv].
SNK_API int snk_mlstm(const float* proj, long long ld, int q_off, int k_off, int v_off, int i_off, int f_off,
                      const void* bias_i, const void* bias_f, int bias_f32, float cap, const int* cu_seqlens,
                      const int* seg_start, const int* seg_slot, float* state_s, float* state_n, float* state_m,
                      float* out, int B, int H, int dk, int dv, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (H <= 0 || H > 65535 || dk <= 0 || dk > 128 || dv <= 0 || dv > 1024 || !(cap > 0.f)) return SNK_ERR_SIZE;
  const int slices = (dv + ML_COLS - 1) / ML_COLS;
  const int warps = ML_TPC * ML_COLS / 32;
  const int dkp = (dk + 4 * ML_TPC - 1) / (4 * ML_TPC) * (4 * ML_TPC);
  const size_t smem = (size_t)(ML_CHUNK * (2 * dkp + ML_COLS + 7)) * sizeof(float);
  dim3 grid(B, H, slices);
#define ML_LAUNCH(DKR_)                                                                                  \
  do {                                                                                                   \
    if (smem > 48 * 1024)                                                                                \
      cudaFuncSetAttribute(mlstm_kernel<DKR_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
    snk_launch(mlstm_kernel<DKR_>, dim3(grid), dim3(warps * 32), smem, stream, proj, ld, q_off, k_off,   \
               v_off, i_off, f_off, SmallVec{bias_i, bias_f32}, SmallVec{bias_f, bias_f32}, cap,         \
               cu_seqlens, seg_start, seg_slot, state_s, state_n, state_m, out, H, dk, dv);              \
  } while (0)
  if (dk <= 32) ML_LAUNCH(32);
  else if (dk <= 64) ML_LAUNCH(64);
  else ML_LAUNCH(128);
#undef ML_LAUNCH
  SNK_LAUNCH_CHECK();
  return 0;
}
