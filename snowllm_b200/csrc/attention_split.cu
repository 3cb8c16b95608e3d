// Windowed grouped-query attention over a paged cache whose keys and values have widths of their own,
// with what the plain kernel (attention.cu) does not have:
//
//   * keys [page, kv head, page_size, maps*dk] and values [page, kv head, page_size, dv] in two pools;
//   * `maps` softmax maps per head over the same values: q is [M, nq, dk] with nq = heads * maps, query
//     head (h, map) reads the key at offset map*dk of kv head h / group, and every map has an output row
//     of its own [M, nq, dv] (a mixer that subtracts one map from another does so afterwards);
//   * a bias per (query head, distance): s = (q . k) * scale + bias[head][min(i - j, bias_len - 1)];
//   * scores, softmax weights and the products with the values in float whatever the cache dtype (the
//     weights are never rounded to 16 bits), output in float or in the compute dtype.
//
// A block serves up to R consecutive rows of one request and one kv head: its warps take (row, query
// head) units in turns, all reading the same tiles of 32 keys and values from shared memory (16-byte
// cp.async, three tiles in flight; rows that are not 16-byte multiples are copied element by element).
// Tiles are aligned to absolute positions, and a unit walks only the tiles that its own window touches,
// in ascending order: what a row computes depends on its position alone, not on the rows beside it.
//
// The first kernel of the file prepares the step's rows: per-head RMS norm of q and k, rotation of the
// first rot_dim elements of each head (split halves; cos and sin times a magnitude), q out, k and v into
// their pages.
#include "common.cuh"

#define SA_TILE 32
#define SA_STAGES 3

template <typename T> struct SaVec;
template <> struct SaVec<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void unpack(const uint4& v, float (&f)[4]) {
    f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y);
    f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
  }
};
template <> struct SaVec<bf16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void unpack(const uint4& v, float (&f)[8]) {
    f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xffff0000u);
    f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xffff0000u);
    f[4] = __uint_as_float(v.z << 16); f[5] = __uint_as_float(v.z & 0xffff0000u);
    f[6] = __uint_as_float(v.w << 16); f[7] = __uint_as_float(v.w & 0xffff0000u);
  }
};

__device__ __forceinline__ void sa_cp_async16(void* smem, const void* gmem, bool valid) {
  const unsigned dst = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void sa_cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N> __device__ __forceinline__ void sa_cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N));
}

// ---------------------------------------------------------------------------------------------
// One warp per (row, head) of q, k and v.  proj: the fused projection's output, row pitch ld, with q at
// column q_off ([nq, dk]), k at k_off ([nkh, dk], nkh = kv heads * maps) and v at v_off ([nkv, dv]).
template <typename T>
__global__ void split_prepare_kernel(const T* __restrict__ proj, long long ld, int q_off, int k_off, int v_off,
                                     SmallVec q_gamma, SmallVec k_gamma, int has_norm, float eps,
                                     const float* __restrict__ inv_freq, int rot_dim, float rot_mult,
                                     const int* __restrict__ positions, const int* __restrict__ row_seg,
                                     const int* __restrict__ block_table, int max_pages, int page_size,
                                     T* __restrict__ kpool, T* __restrict__ vpool, T* __restrict__ q_out,
                                     int nq, int nkh, int nkv, int dk, int dv, int write_kv) {
  pdl_begin();
  extern __shared__ float sp_sh[];                     // [warps][dk]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m = blockIdx.x;
  const int unit = blockIdx.y * (blockDim.x >> 5) + warp;
  const int units = nq + (write_kv ? nkh + nkv : 0);
  if (unit >= units) return;
  const T* row = proj + (size_t)m * ld;
  const int pos = positions[m];
  int page = 0;
  if (unit >= nq) page = block_table[(size_t)row_seg[m] * max_pages + pos / page_size];
  if (unit >= nq + nkh) {                              // a value head: copy
    const int h = unit - nq - nkh;
    const T* src = row + v_off + (size_t)h * dv;
    T* dst = vpool + (((size_t)page * nkv + h) * page_size + pos % page_size) * dv;
    for (int d = lane; d < dv; d += 32) dst[d] = src[d];
    return;
  }
  const bool is_q = unit < nq;
  const int h = is_q ? unit : unit - nq;
  const T* src = row + (is_q ? q_off : k_off) + (size_t)h * dk;
  float* xs = sp_sh + (size_t)warp * dk;
  float ss = 0.f;
  for (int d = lane; d < dk; d += 32) {
    const float v = to_f<T>(src[d]);
    xs[d] = v;
    ss = fmaf(v, v, ss);
  }
  if (has_norm) {
    ss = warp_sum(ss);
    const float inv = 1.f / sqrtf(ss / (float)dk + eps);
    const SmallVec& g = is_q ? q_gamma : k_gamma;
    for (int d = lane; d < dk; d += 32) xs[d] = xs[d] * inv * g[d];
  }
  __syncwarp();
  T* dst;
  if (is_q) {
    dst = q_out + ((size_t)m * nq + h) * dk;
  } else {
    // key head h = kv head * maps + map: the maps of a kv head lie side by side in one row of the pool
    const int maps = nkh / nkv;
    dst = kpool + ((((size_t)page * nkv + h / maps) * page_size + pos % page_size) * maps + h % maps) * dk;
  }
  const int half = rot_dim >> 1;
  for (int d = lane; d < dk; d += 32) {
    float v = xs[d];
    if (d < rot_dim) {
      const int i = d < half ? d : d - half;
      float sn, cs;
      sincosf((float)pos * inv_freq[i], &sn, &cs);
      sn *= rot_mult;
      cs *= rot_mult;
      v = d < half ? xs[d] * cs - xs[d + half] * sn : xs[d] * cs + xs[d - half] * sn;
    }
    dst[d] = from_f<T>(v);
  }
}

SNK_API int snk_split_prepare(const void* proj, long long ld, int q_off, int k_off, int v_off, const void* q_gamma,
                              const void* k_gamma, int gamma_f32, int has_norm, float eps, const float* inv_freq,
                              int rot_dim, float rot_mult, const int* positions, const int* row_seg,
                              const int* block_table, int max_pages, int page_size, void* kpool, void* vpool,
                              void* q_out, int M, int nq, int nkh, int nkv, int dk, int dv, int write_kv, int dtype,
                              cudaStream_t stream) {
  if (M <= 0) return 0;
  if (nq <= 0 || dk <= 0 || rot_dim < 0 || rot_dim > dk || (rot_dim & 1)) return SNK_ERR_SIZE;
  if (write_kv && (nkv <= 0 || nkh <= 0 || nkh % nkv || dv <= 0)) return SNK_ERR_SIZE;
  const int units = nq + (write_kv ? nkh + nkv : 0);
  const int warps = units < 8 ? units : 8;
  dim3 grid(M, (units + warps - 1) / warps);
  const size_t smem = (size_t)warps * dk * sizeof(float);
  if (smem > 48 * 1024) return SNK_ERR_SIZE;
  SNK_DISPATCH(dtype, snk_launch(split_prepare_kernel<T>, dim3(grid), dim3(warps * 32), smem, stream,
                                 static_cast<const T*>(proj), ld, q_off, k_off, v_off,
                                 SmallVec{q_gamma, gamma_f32}, SmallVec{k_gamma, gamma_f32}, has_norm, eps, inv_freq,
                                 rot_dim, rot_mult, positions, row_seg, block_table, max_pages, page_size,
                                 static_cast<T*>(kpool), static_cast<T*>(vpool), static_cast<T*>(q_out), nq, nkh,
                                 nkv, dk, dv, write_kv));
  SNK_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------------------------
// DPL: output elements per lane (dv <= 32 * DPL); UPW: (row, head) units per warp.
template <typename T, int DPL, int UPW>
__global__ void split_attention_kernel(
    const T* __restrict__ q, const T* __restrict__ kpool, const T* __restrict__ vpool,
    const int* __restrict__ block_table, int max_pages, int page_size, const int* __restrict__ positions,
    const int* __restrict__ row_seg, const int* __restrict__ tiles, void* __restrict__ out, int out_f32,
    int nq, int nkv, int maps, int dk, int dv, int window, float scale, const float* __restrict__ bias,
    int bias_len, int vec_ok) {
  pdl_begin();
  extern __shared__ __align__(16) unsigned char sa_raw[];
  constexpr int VEC = SaVec<T>::N;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int m0 = tiles ? tiles[2 * blockIdx.x] : (int)blockIdx.x;
  const int rows = tiles ? tiles[2 * blockIdx.x + 1] : 1;
  const int kvh = blockIdx.y;
  const int hpv = nq / nkv;                              // query heads (maps counted) per kv head
  const int units = rows * hpv;
  const int pos0 = positions[m0];
  const int lo = window > 0 ? max(0, pos0 - window + 1) : 0;
  const int hi = pos0 + rows - 1;                        // the last row's own position
  const int kw = maps * dk;                              // a key row holds the maps side by side

  const int k_bytes = kw * (int)sizeof(T), v_bytes = dv * (int)sizeof(T);
  const int k_stride = ((k_bytes + 15) & ~15) + 16, v_stride = ((v_bytes + 15) & ~15) + 16;
  const int stage_bytes = SA_TILE * (k_stride + v_stride);
  float* qs = reinterpret_cast<float*>(sa_raw + (size_t)SA_STAGES * stage_bytes);

  for (int i = threadIdx.x; i < units * dk; i += blockDim.x) {
    const int u = i / dk, d = i - u * dk;
    const int r = u / hpv, hh = u - r * hpv;
    qs[i] = to_f<T>(q[((size_t)(m0 + r) * nq + kvh * hpv + hh) * dk + d]) * scale;
  }
  const int* bt = block_table + (size_t)row_seg[m0] * max_pages;
  const int t_first = (lo / SA_TILE) * SA_TILE;
  const int ntiles = (hi - t_first) / SA_TILE + 1;

  auto issue = [&](int tile) {
    if (tile < ntiles) {
      const int t0 = t_first + tile * SA_TILE;
      unsigned char* ks = sa_raw + (size_t)(tile % SA_STAGES) * stage_bytes;
      unsigned char* vs = ks + SA_TILE * k_stride;
      if (vec_ok) {
        const int kv_ = k_bytes / 16, vv_ = v_bytes / 16, per = kv_ + vv_;
        for (int v = threadIdx.x; v < SA_TILE * per; v += blockDim.x) {
          const int j = v / per, c = v - j * per;
          const int kp = t0 + j;
          const bool valid = kp >= lo && kp <= hi;
          const T* src = kpool;
          unsigned char* dst = c < kv_ ? ks + j * k_stride + c * 16 : vs + j * v_stride + (c - kv_) * 16;
          if (valid) {
            const size_t slot = ((size_t)bt[kp / page_size] * nkv + kvh) * page_size + kp % page_size;
            src = c < kv_ ? kpool + slot * kw + c * VEC : vpool + slot * dv + (c - kv_) * VEC;
          }
          sa_cp_async16(dst, src, valid);
        }
      } else {
        const int per = kw + dv;
        for (int v = threadIdx.x; v < SA_TILE * per; v += blockDim.x) {
          const int j = v / per, c = v - j * per;
          const int kp = t0 + j;
          T val = from_f<T>(0.f);
          if (kp >= lo && kp <= hi) {
            const size_t slot = ((size_t)bt[kp / page_size] * nkv + kvh) * page_size + kp % page_size;
            val = c < kw ? kpool[slot * kw + c] : vpool[slot * dv + (c - kw)];
          }
          if (c < kw) reinterpret_cast<T*>(ks + j * k_stride)[c] = val;
          else reinterpret_cast<T*>(vs + j * v_stride)[c - kw] = val;
        }
      }
    }
    sa_cp_async_commit();
  };

  float mx[UPW], l[UPW], o[UPW][DPL];
#pragma unroll
  for (int i = 0; i < UPW; ++i) {
    mx[i] = -INFINITY;
    l[i] = 0.f;
#pragma unroll
    for (int e = 0; e < DPL; ++e) o[i][e] = 0.f;
  }

#pragma unroll
  for (int s = 0; s < SA_STAGES - 1; ++s) issue(s);
  for (int tile = 0; tile < ntiles; ++tile) {
    sa_cp_async_wait<SA_STAGES - 2>();
    __syncthreads();                                     // the tile is in (and q, the first time round)
    issue(tile + SA_STAGES - 1);
    const int t0 = t_first + tile * SA_TILE;
    const unsigned char* ks = sa_raw + (size_t)(tile % SA_STAGES) * stage_bytes;
    const unsigned char* vs = ks + SA_TILE * k_stride;
    const int kp = t0 + lane;
#pragma unroll
    for (int i = 0; i < UPW; ++i) {
      const int u = warp + nwarps * i;
      if (u >= units) continue;
      const int r = u / hpv, hh = u - r * hpv;
      const int map = hh % maps;
      const int p = pos0 + r;
      const int klo = window > 0 ? max(0, p - window + 1) : 0;
      if (t0 > p || t0 + SA_TILE - 1 < klo) continue;    // none of this unit's keys in the tile
      const bool valid = kp >= klo && kp <= p;
      const float* qw = qs + (size_t)u * dk;
      float s = 0.f;
      if (vec_ok && dk % VEC == 0) {
        const unsigned char* kr = ks + lane * k_stride + map * dk * (int)sizeof(T);
        for (int cv = 0; cv < dk / VEC; ++cv) {
          float f[VEC];
          SaVec<T>::unpack(*reinterpret_cast<const uint4*>(kr + cv * 16), f);
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
        const T* kr = reinterpret_cast<const T*>(ks + lane * k_stride) + map * dk;
        for (int d = 0; d < dk; ++d) s = fmaf(qw[d], to_f<T>(kr[d]), s);
      }
      if (bias && valid) s += bias[(size_t)(kvh * hpv + hh) * bias_len + min(p - kp, bias_len - 1)];
      s = valid ? s : -INFINITY;
      const float m_new = fmaxf(mx[i], warp_max(s));     // finite: the tile holds a key of this unit
      const float corr = expf(mx[i] - m_new);            // 0 the first time
      const float pw = valid ? expf(s - m_new) : 0.f;
      l[i] = l[i] * corr + warp_sum(pw);
      mx[i] = m_new;
#pragma unroll
      for (int e = 0; e < DPL; ++e) o[i][e] *= corr;
      for (int j = 0; j < SA_TILE; ++j) {
        const float pj = __shfl_sync(0xffffffffu, pw, j);
        const T* vr = reinterpret_cast<const T*>(vs + j * v_stride);
#pragma unroll
        for (int e = 0; e < DPL; ++e) {
          const int d = lane + 32 * e;
          if (d < dv) o[i][e] = fmaf(pj, to_f<T>(vr[d]), o[i][e]);
        }
      }
    }
  }
  sa_cp_async_wait<0>();
#pragma unroll
  for (int i = 0; i < UPW; ++i) {
    const int u = warp + nwarps * i;
    if (u >= units) continue;
    const int r = u / hpv, hh = u - r * hpv;
    const float inv = 1.f / l[i];
    const size_t at = ((size_t)(m0 + r) * nq + kvh * hpv + hh) * dv;
#pragma unroll
    for (int e = 0; e < DPL; ++e) {
      const int d = lane + 32 * e;
      if (d < dv) {
        if (out_f32) static_cast<float*>(out)[at + d] = o[i][e] * inv;
        else static_cast<T*>(out)[at + d] = from_f<T>(o[i][e] * inv);
      }
    }
  }
}

// Rows a block can serve for `hpv` query heads per kv head: the host cuts its tiles to this.
SNK_API int snk_split_attention_tile_rows(int hpv, int decode_only) {
  if (hpv <= 0 || hpv > 32) return 0;
  return decode_only ? 1 : 32 / hpv;
}

// tiles: int32 [num_tiles, 2] = (first row, rows <= tile_rows), consecutive rows of one request; null:
// num_tiles rows, one per block.
SNK_API int snk_split_attention(const void* q, const void* kpool, const void* vpool, const int* block_table,
                                int max_pages, int page_size, const int* positions, const int* row_seg,
                                const int* tiles, int num_tiles, int tile_rows, void* out, int out_f32, int nq,
                                int nkv, int maps, int dk, int dv, int window, float scale, const float* bias,
                                int bias_len, int dtype, cudaStream_t stream) {
  if (num_tiles <= 0) return 0;
  if (nkv <= 0 || maps <= 0 || nq % (nkv * maps) || dk <= 0 || dv <= 0 || dv > 256) return SNK_ERR_SIZE;
  const int hpv = nq / nkv;
  if (hpv > 32 || tile_rows < 1 || tile_rows * hpv > 32 || nkv > 65535) return SNK_ERR_SIZE;
  if (!tiles) tile_rows = 1;
  if (bias && bias_len <= 0) return SNK_ERR_SIZE;
  const int esz = dtype == SNK_F32 ? 4 : 2;
  const int kw = maps * dk;
  const int vec_ok = (kw * esz) % 16 == 0 && (dv * esz) % 16 == 0 && (uintptr_t)kpool % 16 == 0 &&
                     (uintptr_t)vpool % 16 == 0;
  const int cap = tile_rows * hpv;                       // units a block may have to serve
  const int upw = cap > 16 ? 4 : 1;
  const int warps = upw == 1 ? cap : 8;
  const size_t stage = (size_t)SA_TILE * ((((size_t)kw * esz + 15) & ~(size_t)15) + 16 + (((size_t)dv * esz + 15) & ~(size_t)15) + 16);
  const size_t smem = SA_STAGES * stage + (size_t)cap * dk * sizeof(float);
  if (smem > 227 * 1024) return SNK_ERR_SIZE;
  dim3 grid(num_tiles, nkv);
#define SA_LAUNCH(DPL_, UPW_)                                                                          \
  do {                                                                                                 \
    if (smem > 48 * 1024)                                                                              \
      cudaFuncSetAttribute(split_attention_kernel<T, DPL_, UPW_>,                                      \
                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                    \
    snk_launch(split_attention_kernel<T, DPL_, UPW_>, dim3(grid), dim3(warps * 32), smem, stream,      \
               static_cast<const T*>(q), static_cast<const T*>(kpool), static_cast<const T*>(vpool),   \
               block_table, max_pages, page_size, positions, row_seg, tiles, out, out_f32, nq, nkv,    \
               maps, dk, dv, window, scale, bias, bias_len, vec_ok);                                   \
  } while (0)
#define SA_LAUNCH_U(DPL_)                  \
  do {                                     \
    if (upw == 1) SA_LAUNCH(DPL_, 1);      \
    else SA_LAUNCH(DPL_, 4);               \
  } while (0)
  SNK_DISPATCH(dtype, {
    if (dv <= 32) SA_LAUNCH_U(1);
    else if (dv <= 64) SA_LAUNCH_U(2);
    else if (dv <= 128) SA_LAUNCH_U(4);
    else SA_LAUNCH_U(8);
  });
#undef SA_LAUNCH_U
#undef SA_LAUNCH
  SNK_LAUNCH_CHECK();
  return 0;
}
