// Latent attention: every position keeps ONE row for all heads, [c (r), k_rot (rd)]: a low-rank latent of
// the keys and values and one rotated key part that all heads share.  A head's unrotated key is W_uk c and
// its value W_uv c; neither is ever formed.  The query side takes W_uk in (q_abs = W_uk^T q_unrot, r wide),
// so that a head's score is (q_abs . c + q_rot . k_rot) * scale, and the value side leaves the heads'
// weighted sums of c (o_lat, r wide) for the product with W_uv that follows.  Seen from the kernel this is
// attention with one key row of r + rd shared by all heads, whose first r elements are the value.
//
//   latent_prepare:    the step's rows: RMS norm of the latent, rotation of the shared key part and of each
//                      head's rotated query part (pairs (2i, 2i+1), angle position * f_i in float), the row
//                      into its page, q_unrot out head-major (the layout the grouped product reads), q_rot out
//   latent_attention:  CUDA cores, float and bfloat16, any sizes up to r = 512; causal or a window of the
//                      last `window` keys; optionally a sink per head (a term exp(sink) in the softmax's
//                      denominator that has no key and no value); rows alone may have their keys cut into
//                      chunks (merged in chunk order by attention.cu's merge; the sink enters in a row's
//                      first chunk)
//   latent_attention_mma: bfloat16 with r and rd multiples of 16, on mma.sync: what the entry point launches
//                      for those sizes (see there)
//   heads_to_rows:     [heads, M, d] -> [M, heads * d]
//
// Scores, softmax weights, maxima and sums are float whatever the cache dtype.  Key tiles are aligned to
// absolute positions and a (row, head) unit walks only the tiles its own keys lie in, in ascending order:
// what a row computes depends on its position alone.
#include "common.cuh"

#define LA_TILE 32
#define LA_UPW 2
#define LA_MAX_WARPS 8

template <typename T> struct LaVec;
template <> struct LaVec<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void unpack(const uint4& v, float (&f)[4]) {
    f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y);
    f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
  }
};
template <> struct LaVec<bf16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void unpack(const uint4& v, float (&f)[8]) {
    f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xffff0000u);
    f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xffff0000u);
    f[4] = __uint_as_float(v.z << 16); f[5] = __uint_as_float(v.z & 0xffff0000u);
    f[6] = __uint_as_float(v.w << 16); f[7] = __uint_as_float(v.w & 0xffff0000u);
  }
};

__device__ __forceinline__ void la_cp_async16(void* smem, const void* gmem, bool valid) {
  const unsigned dst = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void la_cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N> __device__ __forceinline__ void la_cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N));
}

// Rotation of pairs (2i, 2i+1), i < rot/2, of x[0, n) by the angle pos * inv_freq[i]; the rest passes.
// One warp; xs holds the n values in float.
__device__ __forceinline__ float la_rotated(const float* xs, int d, int rot, int pos, const float* inv_freq) {
  if (d >= rot) return xs[d];
  float sn, cs;
  sincosf((float)pos * inv_freq[d >> 1], &sn, &cs);
  return (d & 1) ? xs[d] * cs + xs[d - 1] * sn : xs[d] * cs - xs[d + 1] * sn;
}

// ---------------------------------------------------------------------------------------------
// One warp per unit of a row: unit h < H is query head h, unit H is the latent row (only with write_kv).
// q: [M, ld_q] with head h at column q_off + h * (dim + rd) as [dim unrotated, rd rotated].
// kv: [M, ld_kv] with the latent at column kv_off as [r, rd].
template <typename T>
__global__ void latent_prepare_kernel(const T* __restrict__ q, long long ld_q, int q_off, const T* __restrict__ kv,
                                      long long ld_kv, int kv_off, SmallVec c_gamma, float eps,
                                      const float* __restrict__ inv_freq, int rot, const int* __restrict__ positions,
                                      const int* __restrict__ row_seg, const int* __restrict__ block_table,
                                      int max_pages, int page_size, T* __restrict__ pool, T* __restrict__ q_unrot,
                                      T* __restrict__ q_rot, int M, int H, int dim, int rd, int r, int write_kv) {
  pdl_begin();
  extern __shared__ float lp_sh[];                     // [warps][max(rd, r + rd)]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m = blockIdx.x;
  const int unit = blockIdx.y * (blockDim.x >> 5) + warp;
  const int units = H + (write_kv ? 1 : 0);
  if (unit >= units) return;
  const int pos = positions[m];
  const int wide = write_kv ? r + rd : rd;
  float* xs = lp_sh + (size_t)warp * wide;
  if (unit < H) {
    const T* src = q + (size_t)m * ld_q + q_off + (size_t)unit * (dim + rd);
    T* dst = q_unrot + ((size_t)unit * M + m) * dim;
    for (int d = lane; d < dim; d += 32) dst[d] = src[d];
    for (int d = lane; d < rd; d += 32) xs[d] = to_f<T>(src[dim + d]);
    __syncwarp();
    T* dr = q_rot + ((size_t)m * H + unit) * rd;
    for (int d = lane; d < rd; d += 32) dr[d] = from_f<T>(la_rotated(xs, d, rot, pos, inv_freq));
    return;
  }
  const T* src = kv + (size_t)m * ld_kv + kv_off;
  float ss = 0.f;
  for (int d = lane; d < r + rd; d += 32) {
    const float v = to_f<T>(src[d]);
    xs[d] = v;
    if (d < r) ss = fmaf(v, v, ss);
  }
  ss = warp_sum(ss);
  const float inv = 1.f / sqrtf(ss / (float)r + eps);
  __syncwarp();
  const int page = block_table[(size_t)row_seg[m] * max_pages + pos / page_size];
  T* dst = pool + ((size_t)page * page_size + pos % page_size) * (r + rd);
  for (int d = lane; d < r; d += 32) dst[d] = from_f<T>(xs[d] * inv * c_gamma[d]);
  for (int d = lane; d < rd; d += 32) dst[r + d] = from_f<T>(la_rotated(xs + r, d, rot, pos, inv_freq));
}

SNK_API int snk_latent_prepare(const void* q, long long ld_q, int q_off, const void* kv, long long ld_kv, int kv_off,
                               const void* c_gamma, int gamma_f32, float eps, const float* inv_freq, int rot,
                               const int* positions, const int* row_seg, const int* block_table, int max_pages,
                               int page_size, void* pool, void* q_unrot, void* q_rot, int M, int H, int dim, int rd,
                               int r, int write_kv, int dtype, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (H <= 0 || dim <= 0 || rd < 0 || r <= 0 || rot < 0 || rot > rd || (rot & 1)) return SNK_ERR_SIZE;
  const int units = H + (write_kv ? 1 : 0);
  const int warps = units < 8 ? units : 8;
  dim3 grid(M, (units + warps - 1) / warps);
  const size_t smem = (size_t)warps * (write_kv ? r + rd : (rd > 0 ? rd : 1)) * sizeof(float);
  if (smem > 48 * 1024) return SNK_ERR_SIZE;
  SNK_DISPATCH(dtype, snk_launch(latent_prepare_kernel<T>, dim3(grid), dim3(warps * 32), smem, stream,
                                 static_cast<const T*>(q), ld_q, q_off, static_cast<const T*>(kv), ld_kv, kv_off,
                                 SmallVec{c_gamma, gamma_f32}, eps, inv_freq, rot, positions, row_seg, block_table,
                                 max_pages, page_size, static_cast<T*>(pool), static_cast<T*>(q_unrot),
                                 static_cast<T*>(q_rot), M, H, dim, rd, r, write_kv));
  SNK_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------------------------
// A block serves up to LA_UPW * warps (row, head) units: `rows` consecutive rows of one request (tiles[b] =
// (first row, rows); no tiles: one row) times the heads [h0, h0 + hpb).  DPL: value elements per lane.
template <typename T, int DPL>
__global__ void latent_attention_kernel(
    const T* __restrict__ q_abs, const T* __restrict__ q_rot, const T* __restrict__ pool,
    const int* __restrict__ block_table, int max_pages, int page_size, const int* __restrict__ positions,
    const int* __restrict__ row_seg, const int* __restrict__ tiles, T* __restrict__ out, int M, int H, int r,
    int rd, int hpb, int window, float scale, const float* __restrict__ sink, int vec_ok, int k_stride, int chunk,
    int num_chunks, float* __restrict__ part_o, float* __restrict__ part_ml) {
  pdl_begin();
  extern __shared__ __align__(16) unsigned char la_raw[];
  constexpr int VEC = LaVec<T>::N;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int m0 = tiles ? tiles[2 * blockIdx.x] : (int)blockIdx.x;
  const int rows = tiles ? tiles[2 * blockIdx.x + 1] : 1;
  const int h0 = blockIdx.y * hpb;
  const int nh = min(hpb, H - h0);
  const int units = rows * nh;
  const int kw = r + rd;
  const int pos0 = positions[m0];
  int lo = window > 0 ? max(0, pos0 - window + 1) : 0;
  int hi = pos0 + rows - 1;                              // the last row's own position
  bool first_chunk = true;
  if (num_chunks > 1) {
    const int cnk = lo / chunk + (int)blockIdx.z;
    if ((long long)cnk * chunk > hi) return;
    first_chunk = blockIdx.z == 0;
    lo = max(lo, cnk * chunk);
    hi = min(hi, (cnk + 1) * chunk - 1);
  }
  const int stage_bytes = LA_TILE * k_stride;
  float* qs = reinterpret_cast<float*>(la_raw + 2 * (size_t)stage_bytes);

  for (int i = threadIdx.x; i < units * kw; i += blockDim.x) {
    const int u = i / kw, d = i - u * kw;
    const int rr = u / nh, h = h0 + (u - rr * nh);
    const float v = d < r ? to_f<T>(q_abs[((size_t)h * M + m0 + rr) * r + d])
                          : to_f<T>(q_rot[((size_t)(m0 + rr) * H + h) * rd + (d - r)]);
    qs[i] = v * scale;
  }
  const int* bt = block_table + (size_t)row_seg[m0] * max_pages;
  const int t_first = (lo / LA_TILE) * LA_TILE;
  const int ntiles = (hi - t_first) / LA_TILE + 1;

  auto issue = [&](int tile) {
    if (tile < ntiles) {
      const int t0 = t_first + tile * LA_TILE;
      unsigned char* ks = la_raw + (size_t)(tile & 1) * stage_bytes;
      if (vec_ok) {
        const int per = kw / VEC;
        for (int v = threadIdx.x; v < LA_TILE * per; v += blockDim.x) {
          const int j = v / per, c = v - j * per;
          const int kp = t0 + j;
          const bool valid = kp >= lo && kp <= hi;
          const T* src = pool;
          if (valid) src = pool + ((size_t)bt[kp / page_size] * page_size + kp % page_size) * kw + c * VEC;
          la_cp_async16(ks + j * k_stride + c * 16, src, valid);
        }
      } else {
        for (int v = threadIdx.x; v < LA_TILE * kw; v += blockDim.x) {
          const int j = v / kw, c = v - j * kw;
          const int kp = t0 + j;
          T val = from_f<T>(0.f);
          if (kp >= lo && kp <= hi) val = pool[((size_t)bt[kp / page_size] * page_size + kp % page_size) * kw + c];
          reinterpret_cast<T*>(ks + j * k_stride)[c] = val;
        }
      }
    }
    la_cp_async_commit();
  };

  float mx[LA_UPW], l[LA_UPW], o[LA_UPW][DPL];
#pragma unroll
  for (int i = 0; i < LA_UPW; ++i) {
    const int u = warp + nwarps * i;
    mx[i] = -INFINITY;
    l[i] = 0.f;
    if (sink && first_chunk && u < units) {              // exp(sink) in the denominator, once per row and head
      mx[i] = sink[h0 + u % nh];
      l[i] = 1.f;
    }
#pragma unroll
    for (int e = 0; e < DPL; ++e) o[i][e] = 0.f;
  }

  issue(0);
  for (int tile = 0; tile < ntiles; ++tile) {
    la_cp_async_wait<0>();
    __syncthreads();                                     // the tile is in (and q, the first time round); the
    issue(tile + 1);                                     // other stage's readers are done
    const int t0 = t_first + tile * LA_TILE;
    const unsigned char* ks = la_raw + (size_t)(tile & 1) * stage_bytes;
    const int kp = t0 + lane;
#pragma unroll
    for (int i = 0; i < LA_UPW; ++i) {
      const int u = warp + nwarps * i;
      if (u >= units) continue;
      const int rr = u / nh;
      const int p = pos0 + rr;
      const int klo = max(lo, window > 0 ? p - window + 1 : 0);
      const int khi = min(p, hi);
      if (t0 > khi || t0 + LA_TILE - 1 < klo) continue;  // none of this unit's keys in the tile
      const bool valid = kp >= klo && kp <= khi;
      const float* qw = qs + (size_t)u * kw;
      float s = 0.f;
      if (vec_ok) {
        const unsigned char* kr = ks + lane * k_stride;
        for (int cv = 0; cv < kw / VEC; ++cv) {
          float f[VEC];
          LaVec<T>::unpack(*reinterpret_cast<const uint4*>(kr + cv * 16), f);
#pragma unroll
          for (int e = 0; e < VEC; e += 4) {
            const float4 q4 = *reinterpret_cast<const float4*>(qw + cv * VEC + e);
            s = fmaf(q4.x, f[e], s);
            s = fmaf(q4.y, f[e + 1], s);
            s = fmaf(q4.z, f[e + 2], s);
            s = fmaf(q4.w, f[e + 3], s);
          }
        }
      } else {
        const T* kr = reinterpret_cast<const T*>(ks + lane * k_stride);
        for (int d = 0; d < kw; ++d) s = fmaf(qw[d], to_f<T>(kr[d]), s);
      }
      s = valid ? s : -INFINITY;
      const float m_new = fmaxf(mx[i], warp_max(s));     // finite: the tile holds a key of this unit
      const float corr = expf(mx[i] - m_new);            // 0 the first time (without a sink)
      const float pw = valid ? expf(s - m_new) : 0.f;
      l[i] = l[i] * corr + warp_sum(pw);
      mx[i] = m_new;
#pragma unroll
      for (int e = 0; e < DPL; ++e) o[i][e] *= corr;
      for (int j = 0; j < LA_TILE; ++j) {
        const float pj = __shfl_sync(0xffffffffu, pw, j);
        const T* vr = reinterpret_cast<const T*>(ks + j * k_stride);
#pragma unroll
        for (int e = 0; e < DPL; ++e) {
          const int d = lane + 32 * e;
          if (d < r) o[i][e] = fmaf(pj, to_f<T>(vr[d]), o[i][e]);
        }
      }
    }
  }
  la_cp_async_wait<0>();
#pragma unroll
  for (int i = 0; i < LA_UPW; ++i) {
    const int u = warp + nwarps * i;
    if (u >= units) continue;
    const int rr = u / nh, h = h0 + (u - rr * nh);
    if (num_chunks > 1) {
      const size_t slot = ((size_t)blockIdx.x * H + h) * num_chunks + blockIdx.z;
#pragma unroll
      for (int e = 0; e < DPL; ++e) {
        const int d = lane + 32 * e;
        if (d < r) part_o[slot * r + d] = o[i][e];
      }
      if (lane == 0) {
        part_ml[slot * 2] = mx[i];
        part_ml[slot * 2 + 1] = l[i];
      }
      continue;
    }
    const float inv = 1.f / l[i];
    T* dst = out + ((size_t)(m0 + rr) * H + h) * r;
#pragma unroll
    for (int e = 0; e < DPL; ++e) {
      const int d = lane + 32 * e;
      if (d < r) dst[d] = from_f<T>(o[i][e] * inv);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// bfloat16 on mma.sync (m16n8k16): a block of 4 * MTB warps (MTB 1, 2 or 4) serves 16 * MTB (row, head) units over tiles of KT
// keys that come in by 16-byte cp.async, two stages.  The four warps of a group share one tile of 16 units.
// Per key tile: (1) S = Q K^T, each warp a quarter of the tile's keys over the whole row width (bfloat16
// products are exact in float, float sums), scaled and left in shared memory; (2) the softmax step in float,
// eight threads per unit: mask, running maximum, weights and their sum, the factor the sums so far shrink
// by; the float weights are split into two bfloat16 terms, p = hi + lo with lo = bf16(p - hi), so that P
// keeps 16 mantissa bits; (3) O = O * factor + P V, each warp a quarter of the value's columns (the value is
// the first r elements of the key row, read transposed by ldmatrix) with both terms of P.  r and rd are
// multiples of 16.  A unit whose keys a tile does not touch leaves the tile with its sums unchanged bit for
// bit, so a row's result does not depend on its neighbours.
#define LM_S_PAD 4              // floats of padding per row of S

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// Four 8 x 8 matrices of 16-bit elements from shared memory, lane L giving the address of row L % 8 of matrix
// L / 8.  Plain: a lane gets elements 2 (L % 4), + 1 of row L / 4 of each matrix; .trans: rows 2 (L % 4), + 1
// of column L / 4.
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* row) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(row);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void* row) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(row);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}

// e^x as 2^(x log2 e) on the special-function unit (two units in the last place; e^-inf = 0)
__device__ __forceinline__ float lm_exp(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x * 1.4426950408889634f));
  return y;
}

// Shared memory of a block, in bytes.
static inline size_t lm_smem(int mtb, int kt, int k_stride) {
  const size_t U = 16 * (size_t)mtb;
  return 2 * (size_t)kt * k_stride + U * k_stride + U * (kt + LM_S_PAD) * 4 + 2 * U * (kt * 2 + 16) + 3 * U * 4;
}

// MTB: tiles of 16 units in the block; KT: keys per tile (32 or 64); NT: tiles of 8 value columns per warp
// (4 * 8 * NT >= r).
template <int MTB, int KT, int NT>
__global__ void __launch_bounds__(128 * MTB, (KT == 32 && MTB == 1) ? 2 : 1) latent_attention_mma_kernel(
    const bf16* __restrict__ q_abs, const bf16* __restrict__ q_rot, const bf16* __restrict__ pool,
    const int* __restrict__ block_table, int max_pages, int page_size, const int* __restrict__ positions,
    const int* __restrict__ row_seg, const int* __restrict__ tiles, bf16* __restrict__ out, int M, int H, int r,
    int rd, int hpb, int window, float scale, const float* __restrict__ sink, int k_stride, int chunk,
    int num_chunks, float* __restrict__ part_o, float* __restrict__ part_ml) {
  pdl_begin();
  extern __shared__ __align__(16) unsigned char lm_raw[];
  constexpr int U = 16 * MTB;                            // unit rows of the block
  constexpr int THREADS = 128 * MTB;
  constexpr int KPT = KT / 8;                            // keys per thread in the softmax step (8 threads a unit)
  constexpr int KPW = KT / 4;                            // keys per warp in S = Q K^T
  constexpr int S_STRIDE = KT + LM_S_PAD;                // floats per row of S
  constexpr int P_STRIDE = KT * 2 + 16;                  // bytes per row of a P term
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wm = warp >> 2, wq = warp & 3;               // this warp's tile of units, and its quarter
  const int m0 = tiles ? tiles[2 * blockIdx.x] : (int)blockIdx.x;
  const int rows = tiles ? tiles[2 * blockIdx.x + 1] : 1;
  const int h0 = blockIdx.y * hpb;
  const int nh = min(hpb, H - h0);
  const int units = rows * nh;
  const int kw = r + rd;
  const int pos0 = positions[m0];
  int lo = window > 0 ? max(0, pos0 - window + 1) : 0;
  int hi = pos0 + rows - 1;
  bool first_chunk = true;
  if (num_chunks > 1) {
    const int cnk = lo / chunk + (int)blockIdx.z;
    if ((long long)cnk * chunk > hi) return;
    first_chunk = blockIdx.z == 0;
    lo = max(lo, cnk * chunk);
    hi = min(hi, (cnk + 1) * chunk - 1);
  }
  const int stage_bytes = KT * k_stride;
  unsigned char* qs = lm_raw + 2 * (size_t)stage_bytes;                  // [U][k_stride]
  float* ss = reinterpret_cast<float*>(qs + (size_t)U * k_stride);        // [U][S_STRIDE]
  unsigned char* p_hi = reinterpret_cast<unsigned char*>(ss + U * S_STRIDE);
  unsigned char* p_lo = p_hi + U * P_STRIDE;
  float* m_s = reinterpret_cast<float*>(p_lo + U * P_STRIDE);             // [U] running maximum
  float* l_s = m_s + U;                                                   // [U] running sum
  float* c_s = l_s + U;                                                   // [U] this tile's factor

  // the units' queries: [absorbed r, rotated rd] per row, zeros for rows beyond the block's units
  const int per = kw / 8;
  for (int u = warp; u < U; u += 4 * MTB) {
    const bf16* a_src = nullptr;
    const bf16* r_src = nullptr;
    if (u < units) {
      const int rr = u / nh, h = h0 + (u - rr * nh);
      a_src = q_abs + ((size_t)h * M + m0 + rr) * r;
      r_src = q_rot + ((size_t)(m0 + rr) * H + h) * rd - r;
    }
    for (int c = lane; c < per; c += 32) {
      uint4 v = make_uint4(0, 0, 0, 0);
      if (a_src) v = *reinterpret_cast<const uint4*>((c * 8 < r ? a_src : r_src) + c * 8);
      *reinterpret_cast<uint4*>(qs + (size_t)u * k_stride + c * 16) = v;
    }
  }
  if (tid < U) {
    const bool with_sink = sink && first_chunk && tid < units;
    m_s[tid] = with_sink ? sink[h0 + tid % nh] : -INFINITY;
    l_s[tid] = with_sink ? 1.f : 0.f;
  }
  const int* bt = block_table + (size_t)row_seg[m0] * max_pages;
  const int t_first = (lo / KT) * KT;
  const int ntiles = (hi - t_first) / KT + 1;

  // a warp brings whole key rows in, the lanes a row's 16-byte pieces.  Tiles start at multiples of KT, so with
  // pages of a multiple of KT keys a tile lies in one page: one look-up and one division per tile, not per row
  const bool one_page = page_size % KT == 0;
  auto issue = [&](int tile) {
    if (tile < ntiles) {
      const int t0 = t_first + tile * KT;
      unsigned char* ks = lm_raw + (size_t)(tile & 1) * stage_bytes;
      const size_t row0 = one_page ? (size_t)bt[t0 / page_size] * page_size + t0 % page_size : 0;
      for (int j = warp; j < KT; j += 4 * MTB) {
        const int kp = t0 + j;
        const bool valid = kp >= lo && kp <= hi;
        const bf16* src = pool;
        if (valid) src = pool + (one_page ? row0 + j : (size_t)bt[kp / page_size] * page_size + kp % page_size) * kw;
        unsigned char* dst = ks + (size_t)j * k_stride;
        for (int c = lane; c < per; c += 32) la_cp_async16(dst + c * 16, valid ? src + c * 8 : src, valid);
      }
    }
    la_cp_async_commit();
  };

  float oacc[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) oacc[nt][e] = 0.f;

  // the softmax step's unit of this thread: eight threads side by side per unit
  const int su = tid >> 3, sub = tid & 7;
  const int s_p = pos0 + (su < units ? su / nh : 0);
  const int col_w = wq * 8 * NT;                          // this warp's first value column

  issue(0);
  for (int tile = 0; tile < ntiles; ++tile) {
    la_cp_async_wait<0>();
    __syncthreads();                                     // the tile is in; the step before is over everywhere
    issue(tile + 1);
    const int t0 = t_first + tile * KT;
    const unsigned char* ks = lm_raw + (size_t)(tile & 1) * stage_bytes;

    // (1) S = Q K^T for this warp's units and its KPW keys
    {
      // two sets of accumulators, for even and odd steps of 16 dimensions: an MMA then waits for the one four
      // (two) instructions back, not for the one right before it
      float sacc[KPW / 8][4], sodd[KPW / 8][4];
#pragma unroll
      for (int n = 0; n < KPW / 8; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) sacc[n][e] = sodd[n][e] = 0.f;
      const unsigned char* q_at = qs + (size_t)(wm * 16 + (lane & 15)) * k_stride + (lane >> 4) * 16;
      const int steps = kw / 16;
      if (KPW == 16) {
        // 16 keys: one load holds the fragments of two tiles of 8 keys for one step of 16 dimensions
        const unsigned char* k_at = ks + (size_t)(wq * 16 + (lane >> 4) * 8 + (lane & 7)) * k_stride + ((lane >> 3) & 1) * 16;
        int kk = 0;
        for (; kk + 1 < steps; kk += 2) {
          uint32_t bk[4], a[4], bk2[4], a2[4];
          ldsm_x4(bk, k_at + kk * 32);
          ldsm_x4(a, q_at + kk * 32);
          ldsm_x4(bk2, k_at + kk * 32 + 32);
          ldsm_x4(a2, q_at + kk * 32 + 32);
          mma_bf16_16816(sacc[0], a, bk[0], bk[1]);
          mma_bf16_16816(sacc[KPW / 8 - 1], a, bk[2], bk[3]);
          mma_bf16_16816(sodd[0], a2, bk2[0], bk2[1]);
          mma_bf16_16816(sodd[KPW / 8 - 1], a2, bk2[2], bk2[3]);
        }
        if (kk < steps) {
          uint32_t bk[4], a[4];
          ldsm_x4(bk, k_at + kk * 32);
          ldsm_x4(a, q_at + kk * 32);
          mma_bf16_16816(sacc[0], a, bk[0], bk[1]);
          mma_bf16_16816(sacc[KPW / 8 - 1], a, bk[2], bk[3]);
        }
      } else {
        // 8 keys: one load holds the fragments for two steps of 16 dimensions
        const unsigned char* k_at = ks + (size_t)(wq * 8 + (lane & 7)) * k_stride + (lane >> 3) * 16;
        int kk = 0;
        for (; kk + 1 < steps; kk += 2) {
          uint32_t bk[4], a[4], a2[4];
          ldsm_x4(bk, k_at + kk * 32);
          ldsm_x4(a, q_at + kk * 32);
          ldsm_x4(a2, q_at + kk * 32 + 32);
          mma_bf16_16816(sacc[0], a, bk[0], bk[1]);
          mma_bf16_16816(sodd[0], a2, bk[2], bk[3]);
        }
        if (kk < steps) {                                 // an odd number of steps: the last load's second half
          uint32_t bk[4], a[4];                           // repeats the step before and is not used
          ldsm_x4(bk, k_at + kk * 32 - ((lane >> 4) ? 32 : 0));
          ldsm_x4(a, q_at + kk * 32);
          mma_bf16_16816(sacc[0], a, bk[0], bk[1]);
        }
      }
#pragma unroll
      for (int n = 0; n < KPW / 8; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) sacc[n][e] += sodd[n][e];
#pragma unroll
      for (int n = 0; n < KPW / 8; ++n) {
        float* at = ss + (wm * 16 + (lane >> 2)) * S_STRIDE + wq * KPW + n * 8 + (lane & 3) * 2;
        at[0] = sacc[n][0] * scale;
        at[1] = sacc[n][1] * scale;
        at[8 * S_STRIDE] = sacc[n][2] * scale;
        at[8 * S_STRIDE + 1] = sacc[n][3] * scale;
      }
    }
    __syncthreads();

    // (2) the softmax step of unit su
    {
      const int klo = max(lo, window > 0 ? s_p - window + 1 : 0);
      const int khi = su < units ? min(s_p, hi) : -1;
      float sv[KPT];
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < KPT; ++j) {
        const int kp = t0 + sub * KPT + j;
        const bool valid = kp >= klo && kp <= khi;
        sv[j] = valid ? ss[su * S_STRIDE + sub * KPT + j] : -INFINITY;
        mx = fmaxf(mx, sv[j]);
      }
#pragma unroll
      for (int o = 4; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      const float m_old = m_s[su];
      const float m_new = fmaxf(m_old, mx);
      const float m_ref = m_new == -INFINITY ? 0.f : m_new;       // nothing seen yet: every term below is e^-inf = 0
      const float corr = lm_exp(m_old - m_ref);                   // e^0 = 1 exactly for a unit the tile does not touch
      float sum = 0.f;
      __nv_bfloat16* ph = reinterpret_cast<__nv_bfloat16*>(p_hi + su * P_STRIDE) + sub * KPT;
      __nv_bfloat16* pl = reinterpret_cast<__nv_bfloat16*>(p_lo + su * P_STRIDE) + sub * KPT;
#pragma unroll
      for (int j = 0; j < KPT; ++j) {
        const float pw = lm_exp(sv[j] - m_ref);
        sum += pw;
        const __nv_bfloat16 hi16 = __float2bfloat16_rn(pw);
        ph[j] = hi16;
        pl[j] = __float2bfloat16_rn(pw - __bfloat162float(hi16));
      }
#pragma unroll
      for (int o = 4; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      __syncwarp();
      if (sub == 0) {
        m_s[su] = m_new;
        l_s[su] = l_s[su] * corr + sum;
        c_s[su] = corr;
      }
    }
    __syncthreads();

    // (3) O = O * factor + P V for this warp's units and columns
    {
      const float c_lo = c_s[wm * 16 + (lane >> 2)], c_hi = c_s[wm * 16 + (lane >> 2) + 8];
      if (!__all_sync(0xffffffffu, c_lo == 1.f && c_hi == 1.f)) {       // no maximum of the warp's units has grown
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          oacc[nt][0] *= c_lo;
          oacc[nt][1] *= c_lo;
          oacc[nt][2] *= c_hi;
          oacc[nt][3] *= c_hi;
        }
      }
      const unsigned char* v_at = ks + (size_t)(((lane >> 3) & 1) * 8 + (lane & 7)) * k_stride + (col_w + (lane >> 4) * 8) * 2;
      const size_t p_at = (size_t)(wm * 16 + (lane & 15)) * P_STRIDE + (lane >> 4) * 16;
#pragma unroll
      for (int kk = 0; kk < KT / 16; ++kk) {
        uint32_t a_hi[4], a_lo[4];
        ldsm_x4(a_hi, p_hi + p_at + kk * 32);
        ldsm_x4(a_lo, p_lo + p_at + kk * 32);
        // 32 columns at a time: eight independent MMAs between an accumulator's two terms
#pragma unroll
        for (int np = 0; np < NT / 2; np += 2) {
          if (col_w + np * 16 >= r) break;                // columns beyond the value (the same for the whole warp)
          uint32_t bv[4], bw[4];
          ldsm_x4_trans(bv, v_at + (size_t)kk * 16 * k_stride + np * 32);
          const bool two = NT >= 4 && col_w + np * 16 + 16 < r;
          if (two) ldsm_x4_trans(bw, v_at + (size_t)kk * 16 * k_stride + np * 32 + 32);
          mma_bf16_16816(oacc[2 * np], a_hi, bv[0], bv[1]);
          mma_bf16_16816(oacc[2 * np + 1], a_hi, bv[2], bv[3]);
          if (two) {
            mma_bf16_16816(oacc[(2 * np + 2) % NT], a_hi, bw[0], bw[1]);
            mma_bf16_16816(oacc[(2 * np + 3) % NT], a_hi, bw[2], bw[3]);
          }
          mma_bf16_16816(oacc[2 * np], a_lo, bv[0], bv[1]);
          mma_bf16_16816(oacc[2 * np + 1], a_lo, bv[2], bv[3]);
          if (two) {
            mma_bf16_16816(oacc[(2 * np + 2) % NT], a_lo, bw[0], bw[1]);
            mma_bf16_16816(oacc[(2 * np + 3) % NT], a_lo, bw[2], bw[3]);
          }
        }
      }
    }
  }
  la_cp_async_wait<0>();
  __syncthreads();

#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int u = wm * 16 + (lane >> 2) + half * 8;
    if (u >= units) continue;
    const int rr = u / nh, h = h0 + (u - rr * nh);
    if (num_chunks > 1) {
      const size_t slot = ((size_t)blockIdx.x * H + h) * num_chunks + blockIdx.z;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int col = col_w + nt * 8 + (lane & 3) * 2;
        if (col < r) {
          part_o[slot * r + col] = oacc[nt][half * 2];
          part_o[slot * r + col + 1] = oacc[nt][half * 2 + 1];
        }
      }
      if (wq == 0 && (lane & 3) == 0) {
        part_ml[slot * 2] = m_s[u];
        part_ml[slot * 2 + 1] = l_s[u];
      }
      continue;
    }
    const float inv = 1.f / l_s[u];
    bf16* dst = out + ((size_t)(m0 + rr) * H + h) * r;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int col = col_w + nt * 8 + (lane & 3) * 2;
      if (col < r)
        *reinterpret_cast<__nv_bfloat162*>(dst + col) =
            __floats2bfloat162_rn(oacc[nt][half * 2] * inv, oacc[nt][half * 2 + 1] * inv);
    }
  }
}

// Whether the tensor-core kernel takes these sizes (bfloat16 only).  SNOWLLM_B200_LATENT_MMA=0 in the
// environment keeps every launch on the CUDA-core kernel (for A/B runs and tests of that path).
static inline bool lm_ok(int r, int rd, int dtype) {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("SNOWLLM_B200_LATENT_MMA");
    on = (e && e[0] == '0') ? 0 : 1;
  }
  return on && dtype == SNK_BF16 && r % 16 == 0 && rd % 16 == 0 && r >= 16 && r <= 512;
}
#define LM_MAX_UNITS 64          // units of a block of 16 warps: four tiles of 16
static inline int lm_heads_per_block(int H) { return H < 32 ? H : 32; }

// Heads a block takes, and the rows of one request it serves beside each other, for H heads.
static inline int la_heads_per_block(int H) { return H < LA_UPW * LA_MAX_WARPS ? H : LA_UPW * LA_MAX_WARPS; }
SNK_API int snk_latent_attention_tile_rows(int H, int r, int rd, int dtype) {
  const int rows = lm_ok(r, rd, dtype) ? LM_MAX_UNITS / lm_heads_per_block(H) : (LA_UPW * LA_MAX_WARPS) / la_heads_per_block(H);
  return rows < 1 ? 1 : rows;
}

SNK_API int snk_latent_attention(const void* q_abs, const void* q_rot, const void* pool, const int* block_table,
                                 int max_pages, int page_size, const int* positions, const int* row_seg,
                                 const int* tiles, int n_tiles, int tile_rows, void* out, int M, int H, int r, int rd,
                                 int window, float scale, const float* sink, int chunk, int num_chunks,
                                 void* scratch, int dtype, cudaStream_t stream) {
  if (M <= 0 || n_tiles <= 0) return 0;
  if (H <= 0 || r <= 0 || rd < 0 || r > 32 * 16) return SNK_ERR_SIZE;
  if (num_chunks < 1 || num_chunks > 65535 || chunk <= 0 || chunk % LA_TILE) return SNK_ERR_SIZE;
  if (num_chunks > 1 && (tiles != nullptr || scratch == nullptr)) return SNK_ERR_SIZE;
  if (lm_ok(r, rd, dtype) && ((uintptr_t)pool % 16) == 0 && ((uintptr_t)q_abs % 16) == 0 &&
      ((uintptr_t)q_rot % 16) == 0) {
    if (chunk % 64) return SNK_ERR_SIZE;
    const int hpb = lm_heads_per_block(H);
    if (tile_rows < 1 || (tiles && tile_rows * hpb > LM_MAX_UNITS)) return SNK_ERR_SIZE;
    const int units_max = (tiles ? tile_rows : 1) * hpb;
    const int mtb = units_max > 32 ? 4 : (units_max > 16 ? 2 : 1);
    const int groups = (H + hpb - 1) / hpb;
    if (groups > 65535) return SNK_ERR_SIZE;
    const int kw = r + rd;
    const int k_stride = kw * 2 + 16;                    // kw * 2 is a multiple of 32: an odd number of 16-byte units
    // keys per tile: 32 where two blocks then fit an SM (rows alone, whose blocks wait for memory most of the
    // time), else 64; SNOWLLM_B200_LATENT_KEYS=32|64 fixes it (A/B runs)
    static int keys_env = -1;
    if (keys_env < 0) {
      const char* e = getenv("SNOWLLM_B200_LATENT_KEYS");
      keys_env = e ? atoi(e) : 0;
    }
    int kt = (!tiles && lm_smem(mtb, 32, k_stride) <= 113 * 1024) ? 32 : 64;
    if (keys_env == 32 || keys_env == 64) kt = keys_env;
    if (mtb == 4 || lm_smem(mtb, kt, k_stride) > 227 * 1024) kt = 32;      // sixteen warps: 32-key tiles only
    const size_t smem = lm_smem(mtb, kt, k_stride);
    if (smem > 227 * 1024) return SNK_ERR_SIZE;
    float* part_o = static_cast<float*>(scratch);
    float* part_ml = part_o ? part_o + (size_t)M * H * num_chunks * r : nullptr;
    dim3 grid(n_tiles, groups, num_chunks);
#define LM_LAUNCH(MTB_, KT_, NT_)                                                                               \
  do {                                                                                                          \
    if (smem > 48 * 1024)                                                                                       \
      cudaFuncSetAttribute(latent_attention_mma_kernel<MTB_, KT_, NT_>,                                         \
                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                             \
    snk_launch(latent_attention_mma_kernel<MTB_, KT_, NT_>, dim3(grid), dim3(128 * MTB_), smem, stream,         \
               static_cast<const bf16*>(q_abs), static_cast<const bf16*>(q_rot), static_cast<const bf16*>(pool),\
               block_table, max_pages, page_size, positions, row_seg, tiles, static_cast<bf16*>(out), M, H, r,  \
               rd, hpb, window, scale, sink, k_stride, chunk, num_chunks, part_o, part_ml);                     \
  } while (0)
#define LM_PICK_NT(MTB_, KT_)                          \
  do {                                                 \
    if (r <= 64) LM_LAUNCH(MTB_, KT_, 2);              \
    else if (r <= 128) LM_LAUNCH(MTB_, KT_, 4);        \
    else if (r <= 256) LM_LAUNCH(MTB_, KT_, 8);        \
    else LM_LAUNCH(MTB_, KT_, 16);                     \
  } while (0)
    if (mtb == 4) LM_PICK_NT(4, 32);
    else if (mtb == 2 && kt == 64) LM_PICK_NT(2, 64);
    else if (mtb == 2) LM_PICK_NT(2, 32);
    else if (kt == 64) LM_PICK_NT(1, 64);
    else LM_PICK_NT(1, 32);
#undef LM_PICK_NT
#undef LM_LAUNCH
    SNK_LAUNCH_CHECK();
    return 0;
  }
  const int hpb = la_heads_per_block(H);
  if (tile_rows < 1 || tile_rows * hpb > LA_UPW * LA_MAX_WARPS) return SNK_ERR_SIZE;
  const int units_max = (tiles ? tile_rows : 1) * hpb;
  const int warps = units_max < LA_MAX_WARPS ? units_max : LA_MAX_WARPS;
  const int groups = (H + hpb - 1) / hpb;
  if (groups > 65535) return SNK_ERR_SIZE;
  const int kw = r + rd;
  const size_t esz = dtype == SNK_F32 ? 4 : 2;
  const int vec_ok = (kw * esz) % 16 == 0 && ((uintptr_t)pool % 16) == 0;
  int k_stride = (int)((kw * esz + 15) & ~(size_t)15) + 16;
  if ((k_stride / 16) % 2 == 0) k_stride += 16;          // an odd number of 16-byte units: rows fall on different banks
  const size_t smem = 2 * (size_t)LA_TILE * k_stride + (size_t)units_max * kw * sizeof(float);
  if (smem > 227 * 1024) return SNK_ERR_SIZE;
  float* part_o = static_cast<float*>(scratch);
  float* part_ml = part_o ? part_o + (size_t)M * H * num_chunks * r : nullptr;
  dim3 grid(n_tiles, groups, num_chunks);
#define LA_LAUNCH(DPL_)                                                                                        \
  SNK_DISPATCH(dtype, {                                                                                        \
    if (smem > 48 * 1024)                                                                                      \
      cudaFuncSetAttribute(latent_attention_kernel<T, DPL_>, cudaFuncAttributeMaxDynamicSharedMemorySize,      \
                           (int)smem);                                                                         \
    snk_launch(latent_attention_kernel<T, DPL_>, dim3(grid), dim3(warps * 32), smem, stream,                   \
               static_cast<const T*>(q_abs), static_cast<const T*>(q_rot), static_cast<const T*>(pool),        \
               block_table, max_pages, page_size, positions, row_seg, tiles, static_cast<T*>(out), M, H, r,    \
               rd, hpb, window, scale, sink, vec_ok, k_stride, chunk, num_chunks, part_o, part_ml);            \
  })
  if (r <= 32) LA_LAUNCH(1);
  else if (r <= 64) LA_LAUNCH(2);
  else if (r <= 128) LA_LAUNCH(4);
  else if (r <= 256) LA_LAUNCH(8);
  else LA_LAUNCH(16);
#undef LA_LAUNCH
  SNK_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void heads_to_rows_kernel(const T* __restrict__ in, T* __restrict__ out, int M, int H, int d) {
  pdl_begin();
  const long long n = (long long)M * H * d;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const int c = (int)(i % d);
    const long long mh = i / d;
    const int h = (int)(mh % H);
    const long long m = mh / H;
    out[i] = in[((size_t)h * M + m) * d + c];
  }
}

SNK_API int snk_heads_to_rows(const void* in, void* out, int M, int H, int d, int dtype, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (H <= 0 || d <= 0) return SNK_ERR_SIZE;
  const long long n = (long long)M * H * d;
  const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  SNK_DISPATCH(dtype, snk_launch(heads_to_rows_kernel<T>, dim3(blocks), dim3(256), 0, stream,
                                 static_cast<const T*>(in), static_cast<T*>(out), M, H, d));
  SNK_LAUNCH_CHECK();
  return 0;
}
