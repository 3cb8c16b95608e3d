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
//   latent_attention_mma: bfloat16 on mma.sync, see there
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

// Heads a block takes, and the rows of one request it serves beside each other, for H heads.
static inline int la_heads_per_block(int H) { return H < LA_UPW * LA_MAX_WARPS ? H : LA_UPW * LA_MAX_WARPS; }
SNK_API int snk_latent_attention_tile_rows(int H) {
  const int rows = (LA_UPW * LA_MAX_WARPS) / la_heads_per_block(H);
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
