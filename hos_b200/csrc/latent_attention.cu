// Attention over a compressed (latent) key/value cache.
//
// Per position the cache keeps one row of D = R + P numbers shared by all heads: the latent c
// (R numbers, RMS-normed) and one rotated key part (P numbers).  A head's key would be
// [W_uk_h c | rotated part] and its value W_uv_h c; neither is ever formed.  The query side
// absorbs W_uk instead:
//     score_h(i, j) = scale * ( (W_uk_h^T q_h)[0:R] . c_j  +  rot(q_h)[R:D] . rot_key_j )
// and the value projection is applied after the weighted sum of latents:
//     out_h(i) = W_uv_h  sum_j p_h(i, j) c_j.
// So every head reads the same D numbers per key (one key/value "head" of size D whose value is
// its first R numbers).  Scores, softmax and the weighted sums are 32-bit quantities whatever the
// storage type is: 32-bit FMA work in latent_attn_kernel, two bfloat16 terms per 32-bit operand on the
// tensor cores in latent_attn_tc_kernel (bfloat16 rows).  Mask: causal with an optional window of the last `window` keys.  Optional
// sink: a learned number per head that joins the softmax's denominator as exp(sink), without a key
// or a value and unscaled.
//
// Kernels: latent_prep (norm of c, rotations, cache write), latent_attn and latent_attn_tc (keys from
// the step's own rows for sequences that start at position 0, or from the paged cache), latent_merge
// (the shares of a row's keys put together), heads_product and heads_product_tc (the per-head products
// W_uk_h^T q_h and W_uv_h o_h as one launch over all heads).
#include "common.cuh"
#include "kv_layout.cuh"
#include "mma_tile.cuh"

namespace hos {

// ---- latent_prep ---------------------------------------------------------------------------
// proj[n] = [ q: H heads of (dq + P) | c_raw: R | key_rot_raw: P ].  Writes
//   kc[n]     = [ rms(c_raw) * w_norm | rot(key_rot_raw) ]                (the row the cache keeps)
//   q_lat[n][h][R : R + P] = rot(q_h[dq : dq + P])                        (32-bit)
// and stores kc[n] at the token's place in the paged cache (rows of D, not permuted).  With kc null the rows hold
// the queries only (a call that reads another call's cache): nothing is normed or stored.
// Rotation: the first rot_dims of the P numbers, pairs (2i, 2i + 1), angle = position * inv_freq[i].
template <typename T>
__global__ void latent_prep_kernel(const T* __restrict__ proj, int proj_stride, int H, int dq, int R, int P,
                                   const float* __restrict__ w_norm, float eps, const float* __restrict__ inv_freq,
                                   int rot_dims, const int* __restrict__ token_pos, const int* __restrict__ token_seq,
                                   const int* __restrict__ seq_slot, const int* __restrict__ seq_len_after,
                                   T* __restrict__ kc, float* __restrict__ q_lat, T* __restrict__ k_pages,
                                   const int* __restrict__ page_table, int table_stride, int ring_pages) {
    pdl_enter();
    extern __shared__ float2 sincos_tab[];      // [rot_dims / 2]
    __shared__ float scratch[32];
    const int n = blockIdx.x;
    const int seq = token_seq[n];
    if (seq < 0) return;
    const int pos = token_pos[n], D = R + P, half = rot_dims >> 1;
    int page = -1;
    if (k_pages != nullptr && !(ring_pages > 0 && pos + ring_pages * kPageTokens < seq_len_after[seq])) {
        const int lp = pos / kPageTokens;
        page = page_table[(size_t)seq_slot[seq] * table_stride + (ring_pages > 0 ? lp % ring_pages : lp)];
    }
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float s, c;
        sincosf((float)pos * inv_freq[i], &s, &c);
        sincos_tab[i] = make_float2(s, c);
    }
    const T* row = proj + (size_t)n * proj_stride;
    const T* craw = row + (size_t)H * (dq + P);
    const bool keys = kc != nullptr;
    float ss = 0.f;
    if (keys)
        for (int d = threadIdx.x; d < R; d += blockDim.x) {
            const float v = to_float(craw[d]);
            ss = fmaf(v, v, ss);
        }
    const float rinv = rsqrtf(block_sum(ss, scratch) / (float)R + eps);      // (also orders sincos_tab)
    T* out = keys ? kc + (size_t)n * D : nullptr;
    T* cached = page >= 0 ? k_pages + ((size_t)page * kPageTokens + pos % kPageTokens) * D : nullptr;
    if (keys)
        for (int d = threadIdx.x; d < R; d += blockDim.x) {
            const T v = from_float<T>(to_float(craw[d]) * rinv * w_norm[d]);
            out[d] = v;
            if (cached) cached[d] = v;
        }
    // the shared rotated key part, then every head's rotated query part: items of one pair (or one
    // unrotated number beyond rot_dims)
    const int per = half + (P - rot_dims);
    for (int it = threadIdx.x; it < (H + (keys ? 1 : 0)) * per; it += blockDim.x) {
        const int who = it / per, j = it - who * per;       // who == H: the key
        const T* src = who == H ? craw + R : row + (size_t)who * (dq + P) + dq;
        float a, b = 0.f;
        int d0;
        const bool pair = j < half;
        if (pair) {
            d0 = 2 * j;
            const float2 sc = sincos_tab[j];
            const float u = to_float(src[d0]), v = to_float(src[d0 + 1]);
            a = u * sc.y - v * sc.x;
            b = v * sc.y + u * sc.x;
        } else {
            d0 = rot_dims + (j - half);
            a = to_float(src[d0]);
        }
        if (who == H) {
            const T ta = from_float<T>(a), tb = from_float<T>(b);
            out[R + d0] = ta;
            if (cached) cached[R + d0] = ta;
            if (pair) {
                out[R + d0 + 1] = tb;
                if (cached) cached[R + d0 + 1] = tb;
            }
        } else {
            float* q = q_lat + ((size_t)n * H + who) * D + R;
            q[d0] = a;
            if (pair) q[d0 + 1] = b;
        }
    }
}

// ---- latent_attn ---------------------------------------------------------------------------
// One block per (QT consecutive rows, group of kHG heads, share of the keys).  Keys come in tiles of kTK
// positions, each row brought to shared memory as 32-bit numbers and used by all QT rows and all heads of the
// block.  Scores: warp = head, lane = key, QT rows at a time.  Weighted sums: a thread owns up to NC columns of
// the latent for all rows and heads of the block.  Rows of a block that belong to different sequences are walked
// one sequence after the other.  With more than one share of the keys (single rows: decoding), every share leaves
// its running maximum, its denominator and its unnormalised sums, and latent_merge puts them together.
constexpr int kHG = 8, kTK = 32, kAttnThreads = 256;

template <typename T, bool PAGED, int NC, int QT>
__global__ void __launch_bounds__(kAttnThreads)
latent_attn_kernel(const float* __restrict__ q_lat, const T* __restrict__ kc, const T* __restrict__ k_pages,
                   const int* __restrict__ page_table, int table_stride, int ring_pages,
                   const float* __restrict__ sink, T* __restrict__ o_lat, float* __restrict__ part_acc,
                   float* __restrict__ part_ml, const int* __restrict__ token_pos,
                   const int* __restrict__ token_seq, const int* __restrict__ cu_seqlens,
                   const int* __restrict__ seq_slot, int row0, int row_end, int H, int R, int D, int Dq, int Dk,
                   float scale, int window) {
    pdl_enter();
    extern __shared__ float smem[];
    float* qs = smem;                          // [QT][kHG][Dq]
    float* ks = qs + QT * kHG * Dq;            // [kTK][Dk]
    float* ps = ks + kTK * Dk;                 // [QT][kTK][kHG] weights of the tile
    float* alpha = ps + QT * kTK * kHG;        // [QT][kHG] what the running sums are scaled by
    float* denom = alpha + QT * kHG;           // [QT][kHG]
    __shared__ int key_row[kTK];               // where each key of the tile lies (-1: none)
    __shared__ int row_seq[QT], row_pos[QT];
    const int n0 = row0 + blockIdx.x * QT, h0 = blockIdx.y * kHG;
    const int split = blockIdx.z, n_splits = gridDim.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nh = min(kHG, H - h0);
    if (tid < QT) {
        const int n = n0 + tid;
        row_seq[tid] = n < row_end ? token_seq[n] : -1;
        row_pos[tid] = n < row_end ? token_pos[n] : 0;
    }
    for (int i = tid; i < QT * kHG * Dq; i += kAttnThreads) {
        const int t = i / (kHG * Dq), rem = i - t * kHG * Dq, h = rem / Dq, d = rem - h * Dq;
        const int n = n0 + t;
        qs[i] = (n < row_end && h < nh && d < D) ? q_lat[((size_t)n * H + h0 + h) * D + d] : 0.f;
    }
    __syncthreads();
    float m_run[QT], l_run[QT];                // of head `warp`, per row (kept by every lane of the warp)
#pragma unroll
    for (int t = 0; t < QT; ++t) {
        m_run[t] = -INFINITY;
        l_run[t] = 0.f;
        if (warp < nh && sink != nullptr && split == 0 && row_seq[t] >= 0) {
            m_run[t] = sink[h0 + warp];
            l_run[t] = 1.f;
        }
    }
    float acc[NC][QT][kHG];
#pragma unroll
    for (int c = 0; c < NC; ++c)
#pragma unroll
        for (int t = 0; t < QT; ++t)
#pragma unroll
            for (int h = 0; h < kHG; ++h) acc[c][t][h] = 0.f;

    for (int g0 = 0; g0 < QT;) {               // the rows of one sequence at a time
        const int seq = row_seq[g0];
        int g1 = g0 + 1;
        while (g1 < QT && row_seq[g1] == seq) ++g1;
        if (seq < 0) {
            g0 = g1;
            continue;
        }
        const int pos_first = row_pos[g0], pos_last = row_pos[g1 - 1];
        const int lo = window > 0 ? max(0, pos_first - window + 1) : 0;
        const int tiles = (pos_last - lo + kTK) / kTK;
        const int per = (tiles + n_splits - 1) / n_splits;
        const int tile_lo = split * per, tile_hi = min(tiles, tile_lo + per);
        const int seq_first = PAGED ? 0 : cu_seqlens[seq];
        const int* table = PAGED ? page_table + (size_t)seq_slot[seq] * table_stride : nullptr;
        for (int tile = tile_lo; tile < tile_hi; ++tile) {
            const int p0 = lo + tile * kTK;
            __syncthreads();                   // the tile before is used up
            if (tid < kTK) {
                const int p = p0 + tid;
                int r = -1;
                if (p <= pos_last) {
                    if (PAGED) {
                        const int lp = p / kPageTokens;
                        r = table[ring_pages > 0 ? lp % ring_pages : lp] * kPageTokens + p % kPageTokens;
                    } else {
                        r = seq_first + p;
                    }
                }
                key_row[tid] = r;
            }
            __syncthreads();
            {
                const T* base = PAGED ? k_pages : kc;
                if (sizeof(T) == 2 && (D & 7) == 0) {          // 16 bytes (8 numbers) at a time
                    const int groups = D >> 3;
                    for (int x = tid; x < kTK * groups; x += kAttnThreads) {
                        const int j = x / groups, gq = x - j * groups;
                        const int r = key_row[j];
                        float* dst = ks + j * Dk + gq * 8;
                        if (r < 0) {
#pragma unroll
                            for (int e = 0; e < 8; ++e) dst[e] = 0.f;
                        } else {
                            const uint4 raw = *reinterpret_cast<const uint4*>(base + (size_t)r * D + gq * 8);
                            const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                dst[2 * e] = __uint_as_float(w[e] << 16);
                                dst[2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u);
                            }
                        }
                    }
                    for (int x = tid; x < kTK * (Dk - D); x += kAttnThreads) ks[(x / (Dk - D)) * Dk + D + x % (Dk - D)] = 0.f;
                } else {
                    for (int j = warp; j < kTK; j += kAttnThreads / 32) {
                        const int r = key_row[j];
                        float* dst = ks + j * Dk;
                        const T* src = base + (size_t)max(r, 0) * D;
                        for (int d = lane; d < Dk; d += 32) dst[d] = (r >= 0 && d < D) ? to_float(src[d]) : 0.f;
                    }
                }
            }
            __syncthreads();
            if (warp < nh) {
                const float4* kv = reinterpret_cast<const float4*>(ks + lane * Dk);
                float s[QT];
#pragma unroll
                for (int t = 0; t < QT; ++t) s[t] = 0.f;
                for (int i = 0; i < (Dq >> 2); ++i) {
                    const float4 b = kv[i];
#pragma unroll
                    for (int t = 0; t < QT; ++t) {
                        const float4 a = reinterpret_cast<const float4*>(qs + (t * kHG + warp) * Dq)[i];
                        s[t] = fmaf(a.x, b.x, s[t]);
                        s[t] = fmaf(a.y, b.y, s[t]);
                        s[t] = fmaf(a.z, b.z, s[t]);
                        s[t] = fmaf(a.w, b.w, s[t]);
                    }
                }
                const int kp = p0 + lane;
#pragma unroll
                for (int t = 0; t < QT; ++t) {
                    const bool in_group = t >= g0 && t < g1;
                    const int pt = row_pos[t];
                    const bool live = in_group && kp <= pt && (window <= 0 || kp > pt - window);
                    const float sv = live ? s[t] * scale : -INFINITY;
                    const float m_new = fmaxf(m_run[t], warp_max(sv));
                    const float p = live ? expf(sv - m_new) : 0.f;
                    const float a = m_new == -INFINITY ? 1.f : (m_run[t] == -INFINITY ? 0.f : expf(m_run[t] - m_new));
                    l_run[t] = fmaf(l_run[t], a, warp_sum(p));
                    m_run[t] = m_new;
                    ps[(t * kTK + lane) * kHG + warp] = p;
                    if (lane == 0) alpha[t * kHG + warp] = a;
                }
            } else if (warp < kHG) {
#pragma unroll
                for (int t = 0; t < QT; ++t) {
                    ps[(t * kTK + lane) * kHG + warp] = 0.f;
                    if (lane == 0) alpha[t * kHG + warp] = 1.f;
                }
            }
            __syncthreads();
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                const int col = tid + c * kAttnThreads;
                if (col < R) {
#pragma unroll
                for (int t = 0; t < QT; ++t)
#pragma unroll
                    for (int h = 0; h < kHG; ++h) acc[c][t][h] *= alpha[t * kHG + h];
#pragma unroll 2
                for (int j = 0; j < kTK; ++j) {
                    const float v = ks[j * Dk + col];
#pragma unroll
                    for (int t = 0; t < QT; ++t) {
                        const float4 pa = *reinterpret_cast<const float4*>(ps + (t * kTK + j) * kHG);
                        const float4 pb = *reinterpret_cast<const float4*>(ps + (t * kTK + j) * kHG + 4);
                        acc[c][t][0] = fmaf(pa.x, v, acc[c][t][0]);
                        acc[c][t][1] = fmaf(pa.y, v, acc[c][t][1]);
                        acc[c][t][2] = fmaf(pa.z, v, acc[c][t][2]);
                        acc[c][t][3] = fmaf(pa.w, v, acc[c][t][3]);
                        acc[c][t][4] = fmaf(pb.x, v, acc[c][t][4]);
                        acc[c][t][5] = fmaf(pb.y, v, acc[c][t][5]);
                        acc[c][t][6] = fmaf(pb.z, v, acc[c][t][6]);
                        acc[c][t][7] = fmaf(pb.w, v, acc[c][t][7]);
                    }
                }
                }
            }
        }
        g0 = g1;
    }
    __syncthreads();
    if (warp < kHG && lane == 0) {
#pragma unroll
        for (int t = 0; t < QT; ++t) {
            denom[t * kHG + warp] = warp < nh ? l_run[t] : 1.f;
            if (n_splits > 1 && warp < nh && n0 + t < row_end) {
                float* ml = part_ml + (((size_t)(n0 + t) * H + h0 + warp) * n_splits + split) * 2;
                ml[0] = m_run[t];
                ml[1] = l_run[t];
            }
        }
    }
    __syncthreads();
#pragma unroll
    for (int c = 0; c < NC; ++c) {
        const int col = tid + c * kAttnThreads;
        if (col >= R) continue;
#pragma unroll
        for (int t = 0; t < QT; ++t) {
            const int n = n0 + t;
            if (n >= row_end) continue;
#pragma unroll
            for (int h = 0; h < kHG; ++h) {
                if (h >= nh) continue;
                if (n_splits > 1) {
                    part_acc[(((size_t)n * H + h0 + h) * n_splits + split) * R + col] = acc[c][t][h];
                } else {
                    const float d = denom[t * kHG + h];
                    o_lat[((size_t)n * H + h0 + h) * R + col] = from_float<T>((row_seq[t] >= 0 && d > 0.f) ? acc[c][t][h] / d : 0.f);
                }
            }
        }
    }
}

// ---- latent_attn on the tensor cores (bfloat16 rows) -----------------------------------------------
// The same walk with both products as m16n8k16 MMAs.  A block's 16 MMA rows are (2 rows of the step) x (8 heads).
// The 32-bit absorbed query and the 32-bit softmax weights enter the tensor cores as two bfloat16 terms each
// (value = hi + lo, 16 bits of mantissa between them; the keys and latents are bfloat16 as stored), and every
// product is accumulated in 32-bit, so scores and weighted sums stay 32-bit quantities.  Key tiles of 32 positions
// are copied as they lie (16-byte asynchronous copies, two stages, the next tile on its way during the
// arithmetic); rows are padded so that ldmatrix finds no bank conflicts.  Scores: every warp takes a share of the
// row's numbers (16 at a time) for all 32 keys, so that a query fragment is loaded once for four key tiles; the
// shares are added by the softmax warps (two MMA rows each, a lane per key).  Weighted sums: every warp owns NT
// 8-wide column tiles of the latent.
template <bool PAGED, int NT>
__global__ void __launch_bounds__(kAttnThreads)
latent_attn_tc_kernel(const float* __restrict__ q_lat, const bf16* __restrict__ kc, const bf16* __restrict__ k_pages,
                      const int* __restrict__ page_table, int table_stride, int ring_pages,
                      const float* __restrict__ sink, bf16* __restrict__ o_lat, float* __restrict__ part_acc,
                      float* __restrict__ part_ml, const int* __restrict__ token_pos,
                      const int* __restrict__ token_seq, const int* __restrict__ cu_seqlens,
                      const int* __restrict__ seq_slot, int row0, int row_end, int QT, int H, int R, int D, int Ds,
                      float scale, int window) {
    pdl_enter();
    constexpr int kPs = 40, kSs = 36;           // row strides of the weight tiles (bf16) and the partial scores (f32)
    extern __shared__ __align__(128) unsigned char raw[];
    bf16* Qh = reinterpret_cast<bf16*>(raw);    // [16][Ds]
    bf16* Ql = Qh + 16 * Ds;                    // [16][Ds]
    bf16* Kt = Ql + 16 * Ds;                    // [2][kTK][Ds]
    bf16* Ph = Kt + 2 * kTK * Ds;               // [16][kPs]
    bf16* Pl = Ph + 16 * kPs;
    float* Sp = reinterpret_cast<float*>(Pl + 16 * kPs);      // [warps][16][kSs] every warp's share of the scores
    float* alpha = Sp + (kAttnThreads / 32) * 16 * kSs;       // [16]
    float* denom = alpha + 16;                  // [16]
    __shared__ int row_seq[2], row_pos[2];
    const int n0 = row0 + blockIdx.x * QT, h0 = blockIdx.y * kHG;
    const int split = blockIdx.z, n_splits = gridDim.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nh = min(kHG, H - h0);
    if (tid < 2) {
        const int n = n0 + tid;
        const bool in = tid < QT && n < row_end;
        row_seq[tid] = in ? token_seq[n] : -1;
        row_pos[tid] = in ? token_pos[n] : 0;
    }
    for (int i = tid; i < 16 * Ds; i += kAttnThreads) {
        const int row = i / Ds, d = i - row * Ds, t = row >> 3, h = row & 7, n = n0 + t;
        const float v = (t < QT && n < row_end && h < nh && d < D) ? q_lat[((size_t)n * H + h0 + h) * D + d] : 0.f;
        const bf16 hi = __float2bfloat16_rn(v);
        Qh[i] = hi;
        Ql[i] = __float2bfloat16_rn(v - __bfloat162float(hi));
    }
    for (int i = tid; i < 2 * kTK * (Ds - D); i += kAttnThreads)       // the padding columns stay zero
        Kt[(i / (Ds - D)) * Ds + D + i % (Ds - D)] = __float2bfloat16_rn(0.f);
    __syncthreads();
    // the softmax warps' running maxima and denominators: warp w keeps MMA rows 2w and 2w + 1
    float m_run[2], l_run[2];
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        const int row = 2 * warp + rr, t = row >> 3, h = row & 7;
        m_run[rr] = -INFINITY;
        l_run[rr] = 0.f;
        if (h < nh && sink != nullptr && split == 0 && row_seq[t] >= 0) {
            m_run[rr] = sink[h0 + h];
            l_run[rr] = 1.f;
        }
    }
    float acc[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[i][c] = 0.f;
    const int groups = D >> 3;                  // 16-byte groups per stored row
    const int ksteps = (D + 15) >> 4;

    for (int g0 = 0; g0 < 2;) {                 // the rows of one sequence at a time
        const int seq = row_seq[g0];
        int g1 = g0 + 1;
        while (g1 < 2 && row_seq[g1] == seq) ++g1;
        if (seq < 0) {
            g0 = g1;
            continue;
        }
        const int pos_first = row_pos[g0], pos_last = row_pos[g1 - 1];
        const int lo = window > 0 ? max(0, pos_first - window + 1) : 0;
        const int tiles = (pos_last - lo + kTK) / kTK;
        const int per = (tiles + n_splits - 1) / n_splits;
        const int tile_lo = split * per, tile_hi = min(tiles, tile_lo + per);
        const int seq_first = PAGED ? 0 : cu_seqlens[seq];
        const int* table = PAGED ? page_table + (size_t)seq_slot[seq] * table_stride : nullptr;
        const bf16* base = PAGED ? k_pages : kc;
        auto issue = [&](int tile, int stage) {
            const int p0 = lo + tile * kTK;
            bf16* dst = Kt + stage * kTK * Ds;
            for (int x = tid; x < kTK * groups; x += kAttnThreads) {
                const int j = x / groups, gq = x - j * groups, p = p0 + j;
                const bool ok = p <= pos_last;
                size_t r = 0;
                if (ok) {
                    if (PAGED) {
                        const int lp = p / kPageTokens;
                        r = (size_t)table[ring_pages > 0 ? lp % ring_pages : lp] * kPageTokens + p % kPageTokens;
                    } else {
                        r = (size_t)(seq_first + p);
                    }
                }
                cp_async16(dst + j * Ds + gq * 8, base + r * D + gq * 8, ok);
            }
        };
        if (tile_lo < tile_hi) issue(tile_lo, 0);
        cp_async_commit();
        for (int tile = tile_lo; tile < tile_hi; ++tile) {
            const int stage = (tile - tile_lo) & 1, p0 = lo + tile * kTK;
            if (tile + 1 < tile_hi) issue(tile + 1, stage ^ 1);
            cp_async_commit();
            cp_async_wait<1>();
            __syncthreads();
            const bf16* K = Kt + stage * kTK * Ds;
            {   // scores of all 32 keys over this warp's share of the row's numbers (16 at a time, warp after warp)
                float s4[4][4];
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int c = 0; c < 4; ++c) s4[i][c] = 0.f;
                const int arow = (lane & 7) + ((lane >> 3) & 1) * 8, acol = (lane >> 4) * 8;
                const int brow = (lane & 7) + (lane >> 4) * 8, bcol = ((lane >> 3) & 1) * 8;
                for (int ks = warp; ks < ksteps; ks += kAttnThreads / 32) {
                    uint32_t ah[4], al[4], w0[4], w1[4];
                    ldmatrix_x4(ah, smem_u32(Qh + arow * Ds + ks * 16 + acol));
                    ldmatrix_x4(al, smem_u32(Ql + arow * Ds + ks * 16 + acol));
                    ldmatrix_x4(w0, smem_u32(K + brow * Ds + ks * 16 + bcol));
                    ldmatrix_x4(w1, smem_u32(K + (16 + brow) * Ds + ks * 16 + bcol));
                    mma_bf16(s4[0], ah, w0[0], w0[1]);
                    mma_bf16(s4[1], ah, w0[2], w0[3]);
                    mma_bf16(s4[2], ah, w1[0], w1[1]);
                    mma_bf16(s4[3], ah, w1[2], w1[3]);
                    mma_bf16(s4[0], al, w0[0], w0[1]);
                    mma_bf16(s4[1], al, w0[2], w0[3]);
                    mma_bf16(s4[2], al, w1[0], w1[1]);
                    mma_bf16(s4[3], al, w1[2], w1[3]);
                }
                float* out = Sp + warp * 16 * kSs + (lane & 3) * 2;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    *reinterpret_cast<float2*>(out + (lane >> 2) * kSs + i * 8) = make_float2(s4[i][0], s4[i][1]);
                    *reinterpret_cast<float2*>(out + ((lane >> 2) + 8) * kSs + i * 8) = make_float2(s4[i][2], s4[i][3]);
                }
            }
            __syncthreads();
#pragma unroll
            for (int rr = 0; rr < 2; ++rr) {    // softmax of MMA rows 2w, 2w + 1: a lane per key
                const int row = 2 * warp + rr, t = row >> 3, h = row & 7;
                const int kp = p0 + lane, pt = row_pos[t];
                const bool live = t >= g0 && t < g1 && h < nh && kp <= pt && (window <= 0 || kp > pt - window);
                float dot = 0.f;
#pragma unroll
                for (int w = 0; w < kAttnThreads / 32; ++w) dot += Sp[(w * 16 + row) * kSs + lane];
                const float sv = live ? dot * scale : -INFINITY;
                const float m_new = fmaxf(m_run[rr], warp_max(sv));
                const float p = live ? expf(sv - m_new) : 0.f;
                const float a = m_new == -INFINITY ? 1.f : (m_run[rr] == -INFINITY ? 0.f : expf(m_run[rr] - m_new));
                l_run[rr] = fmaf(l_run[rr], a, warp_sum(p));
                m_run[rr] = m_new;
                const bf16 hi = __float2bfloat16_rn(p);
                Ph[row * kPs + lane] = hi;
                Pl[row * kPs + lane] = __float2bfloat16_rn(p - __bfloat162float(hi));
                if (lane == 0) alpha[row] = a;
            }
            __syncthreads();
            {   // weighted sums: this warp's column tiles of the latent
                const float a0 = alpha[lane >> 2], a1 = alpha[(lane >> 2) + 8];
#pragma unroll
                for (int i = 0; i < NT; ++i) {
                    acc[i][0] *= a0;
                    acc[i][1] *= a0;
                    acc[i][2] *= a1;
                    acc[i][3] *= a1;
                }
                const int arow = (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
                for (int kk = 0; kk < 2; ++kk) {
                    uint32_t ph[4], pl[4];
                    ldmatrix_x4(ph, smem_u32(Ph + arow * kPs + kk * 16 + (lane >> 4) * 8));
                    ldmatrix_x4(pl, smem_u32(Pl + arow * kPs + kk * 16 + (lane >> 4) * 8));
#pragma unroll
                    for (int i = 0; i < NT; i += 2) {
                        uint32_t v[4];
                        ldmatrix_x4_trans(v, smem_u32(K + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * Ds +
                                                      (warp * NT + i) * 8 + (lane >> 4) * 8));
                        mma_bf16(acc[i], ph, v[0], v[1]);
                        mma_bf16(acc[i], pl, v[0], v[1]);
                        mma_bf16(acc[i + 1], ph, v[2], v[3]);
                        mma_bf16(acc[i + 1], pl, v[2], v[3]);
                    }
                }
            }
            __syncthreads();                    // the stage is free for the tile after the next
        }
        cp_async_wait<0>();
        g0 = g1;
    }
    __syncthreads();
    if (lane == 0) {
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
            const int row = 2 * warp + rr, t = row >> 3, h = row & 7, n = n0 + t;
            denom[row] = l_run[rr];
            if (n_splits > 1 && h < nh && t < QT && n < row_end) {
                float* ml = part_ml + (((size_t)n * H + h0 + h) * n_splits + split) * 2;
                ml[0] = m_run[rr];
                ml[1] = l_run[rr];
            }
        }
    }
    __syncthreads();
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int row = (lane >> 2) + half * 8, t = row >> 3, h = row & 7, n = n0 + t;
        if (t >= QT || n >= row_end || h >= nh) continue;
        const float d = denom[row];
        const bool live = row_seq[t] >= 0 && d > 0.f;
#pragma unroll
        for (int i = 0; i < NT; ++i) {
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const int col = (warp * NT + i) * 8 + (lane & 3) * 2 + c;
                if (col >= R) continue;
                const float v = acc[i][half * 2 + c];
                if (n_splits > 1) part_acc[(((size_t)n * H + h0 + h) * n_splits + split) * R + col] = v;
                else o_lat[((size_t)n * H + h0 + h) * R + col] = __float2bfloat16_rn(live ? v / d : 0.f);
            }
        }
    }
}

// o_lat[n][h] = sum_s e^{m_s - M} acc_s / sum_s e^{m_s - M} l_s over the shares s of the keys.
template <typename T>
__global__ void latent_merge_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                    T* __restrict__ o_lat, const int* __restrict__ token_seq, int row0, int H, int R,
                                    int n_splits) {
    pdl_enter();
    const int n = row0 + blockIdx.x, h = blockIdx.y;
    T* out = o_lat + ((size_t)n * H + h) * R;
    if (token_seq[n] < 0) {
        for (int c = threadIdx.x; c < R; c += blockDim.x) out[c] = from_float<T>(0.f);
        return;
    }
    const float* ml = part_ml + ((size_t)n * H + h) * n_splits * 2;
    float M = -INFINITY;
    for (int s = 0; s < n_splits; ++s) M = fmaxf(M, ml[2 * s]);
    float den = 0.f;
    for (int s = 0; s < n_splits; ++s) den += ml[2 * s] == -INFINITY ? 0.f : expf(ml[2 * s] - M) * ml[2 * s + 1];
    const float* pa = part_acc + ((size_t)n * H + h) * n_splits * R;
    for (int c = threadIdx.x; c < R; c += blockDim.x) {
        float v = 0.f;
        for (int s = 0; s < n_splits; ++s)
            if (ml[2 * s] != -INFINITY) v = fmaf(expf(ml[2 * s] - M), pa[(size_t)s * R + c], v);
        out[c] = from_float<T>(den > 0.f ? v / den : 0.f);
    }
}

// ---- heads_product -------------------------------------------------------------------------
// out[n, h, o] = sum_i W[h][o][i] * in[n, h, i] for every head h in one launch (blockIdx.z = head):
// 64 x 64 tiles, 32-bit FMA.  Row and head strides of `in` and `out` are given in elements.
template <typename TA, typename TW, typename TO>
__global__ void __launch_bounds__(256)
heads_product_kernel(const TA* __restrict__ A, const TW* __restrict__ W, TO* __restrict__ out, int M, int N, int K,
                     int lda, int a_head, int w_head, int ldo, int o_head) {
    pdl_enter();
    constexpr int BM = 64, BN = 64, BK = 16;
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN, h = blockIdx.z;
    A += (size_t)h * a_head;
    W += (size_t)h * w_head;
    out += (size_t)h * o_head;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += BK) {
        for (int e = threadIdx.x; e < BM * BK; e += 256) {
            const int r = e >> 4, kk = e & 15;
            const int m = m0 + r, k = k0 + kk, nn = n0 + r;
            As[kk][r] = (m < M && k < K) ? to_float(A[(size_t)m * lda + k]) : 0.f;
            Ws[kk][r] = (nn < N && k < K) ? to_float(W[(size_t)nn * K + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int nn = n0 + tx * 4 + j;
            if (nn < N) out[(size_t)m * ldo + nn] = from_float<TO>(acc[i][j]);
        }
    }
}

// The same product for bfloat16 operands on the tensor cores (rows and heads 16-byte aligned, K a multiple of 8).
template <typename TO>
__global__ void __launch_bounds__(256)
heads_product_tc_kernel(const bf16* __restrict__ A, const bf16* __restrict__ W, TO* __restrict__ out, int M, int N, int K,
                        int lda, int a_head, int ldo, int o_head) {
    pdl_enter();
    extern __shared__ __align__(128) unsigned char raw[];
    bf16* smem = reinterpret_cast<bf16*>(raw);
    const int m0 = blockIdx.y * kTile, n0 = blockIdx.x * kTile, h = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warp_m = warp & 3, warp_n = warp >> 2;
    const bf16* Ah = A + (size_t)h * a_head;
    const bool busy = m0 + warp_m * 16 < M;
    float acc[1][4][4] = {};
    tc_mainloop<1>(smem, [&](int r) { return m0 + r < M ? Ah + (size_t)(m0 + r) * lda : (const bf16*)nullptr; },
                   W + (size_t)h * N * K, N, n0, 0, K, busy, acc);
    if (!busy) return;
    TO* Oh = out + (size_t)h * o_head;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int m = m0 + warp_m * 16 + (lane >> 2) + half * 8;
        if (m >= M) continue;
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            const int n = n0 + warp_n * 32 + nt * 8 + (lane & 3) * 2;
#pragma unroll
            for (int c = 0; c < 2; ++c)
                if (n + c < N) Oh[(size_t)m * ldo + n + c] = from_float<TO>(acc[0][nt][half * 2 + c]);
        }
    }
}

template <typename T>
static int launch_prep(const void* proj, int proj_stride, int H, int dq, int R, int P, const float* w_norm, float eps,
                       const float* inv_freq, int rot_dims, const int* token_pos, const int* token_seq,
                       const int* seq_slot, const int* seq_len_after, void* kc, float* q_lat, void* k_pages,
                       const int* page_table, int table_stride, int ring_pages, int N, cudaStream_t stream) {
    launch_pdl(latent_prep_kernel<T>, dim3(N), dim3(128), (size_t)(rot_dims / 2 + 1) * sizeof(float2), stream,
               (const T*)proj, proj_stride, H, dq, R, P, w_norm, eps, inv_freq, rot_dims, token_pos, token_seq, seq_slot,
               seq_len_after, (T*)kc, q_lat, (T*)k_pages, page_table, table_stride, ring_pages);
    return check_launch("latent_prep");
}

template <typename T, bool PAGED, int NC, int QT>
static int launch_attn_as(const float* q_lat, const void* kc, const void* k_pages, const int* page_table, int table_stride,
                          int ring_pages, const float* sink, void* o_lat, float* part_acc, float* part_ml, int n_splits,
                          const int* token_pos, const int* token_seq, const int* cu_seqlens, const int* seq_slot, int row0,
                          int rows, int H, int R, int D, float scale, int window, cudaStream_t stream) {
    const int Dq = (D + 3) / 4 * 4;
    const int Dk = 4 * (((D + 3) / 4) | 1);        // rows of 16-byte groups, an odd number of them: no bank conflicts
    const size_t smem = (size_t)(QT * kHG * Dq + kTK * Dk + QT * kTK * kHG + 2 * QT * kHG) * sizeof(float);
    if (smem > 200 * 1024) HOS_REFUSE("latent_attn: rows of %d numbers do not fit a block's shared memory", D);
    auto kernel = latent_attn_kernel<T, PAGED, NC, QT>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_pdl(kernel, dim3((rows + QT - 1) / QT, (H + kHG - 1) / kHG, n_splits), dim3(kAttnThreads), smem, stream, q_lat,
               (const T*)kc, (const T*)k_pages, page_table, table_stride, ring_pages, sink, (T*)o_lat, part_acc, part_ml,
               token_pos, token_seq, cu_seqlens, seq_slot, row0, row0 + rows, H, R, D, Dq, Dk, scale, window);
    int rc = check_launch("latent_attn");
    if (rc == 0 && n_splits > 1) {
        launch_pdl(latent_merge_kernel<T>, dim3(rows, H), dim3(128), 0, stream, (const float*)part_acc, (const float*)part_ml,
                   (T*)o_lat, token_seq, row0, H, R, n_splits);
        rc = check_launch("latent_merge");
    }
    return rc;
}

template <bool PAGED, int NT>
static int launch_attn_tc_as(const float* q_lat, const void* kc, const void* k_pages, const int* page_table, int table_stride,
                             int ring_pages, const float* sink, void* o_lat, float* part_acc, float* part_ml, int n_splits,
                             int QT, const int* token_pos, const int* token_seq, const int* cu_seqlens, const int* seq_slot,
                             int row0, int rows, int H, int R, int D, float scale, int window, cudaStream_t stream) {
    const int Ds = max((D + 15) / 16 * 16, 64 * NT) + 8;       // rows of 16-byte groups, an odd number of them
    const size_t smem = (size_t)(2 * 16 * Ds + 2 * kTK * Ds + 2 * 16 * 40) * 2 + (size_t)(8 * 16 * 36 + 32) * 4;
    if (smem > 200 * 1024) return 1;                     // does not fit: the caller takes the other kernel
    auto kernel = latent_attn_tc_kernel<PAGED, NT>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_pdl(kernel, dim3((rows + QT - 1) / QT, (H + kHG - 1) / kHG, n_splits), dim3(kAttnThreads), smem, stream, q_lat,
               (const bf16*)kc, (const bf16*)k_pages, page_table, table_stride, ring_pages, sink, (bf16*)o_lat, part_acc,
               part_ml, token_pos, token_seq, cu_seqlens, seq_slot, row0, row0 + rows, QT, H, R, D, Ds, scale, window);
    int rc = check_launch("latent_attn");
    if (rc == 0 && n_splits > 1) {
        launch_pdl(latent_merge_kernel<bf16>, dim3(rows, H), dim3(128), 0, stream, (const float*)part_acc,
                   (const float*)part_ml, (bf16*)o_lat, token_seq, row0, H, R, n_splits);
        rc = check_launch("latent_merge");
    }
    return rc;
}

// 0: launched; 1: not a case for the tensor-core kernel; negative: an error.
template <bool PAGED>
static int launch_attn_tc(const float* q_lat, const void* kc, const void* k_pages, const int* page_table, int table_stride,
                          int ring_pages, const float* sink, void* o_lat, float* part_acc, float* part_ml, int n_splits,
                          int rows_per_block, const int* token_pos, const int* token_seq, const int* cu_seqlens,
                          const int* seq_slot, int row0, int rows, int H, int R, int D, float scale, int window,
                          cudaStream_t stream) {
    const void* src = PAGED ? k_pages : kc;
    if ((D & 7) != 0 || ((uintptr_t)src & 15) != 0 || R > 1024) return 1;
    const int QT = (rows_per_block > 1 && n_splits == 1) ? 2 : 1;
#define HOS_TC(NT) return launch_attn_tc_as<PAGED, NT>(q_lat, kc, k_pages, page_table, table_stride, ring_pages, sink, o_lat,   \
                                                       part_acc, part_ml, n_splits, QT, token_pos, token_seq, cu_seqlens,    \
                                                       seq_slot, row0, rows, H, R, D, scale, window, stream)
    if (R <= 128) HOS_TC(2);
    if (R <= 256) HOS_TC(4);
    if (R <= 512) HOS_TC(8);
    HOS_TC(16);
#undef HOS_TC
}

// Rows per block: four where many rows share keys (prompts), fewer where the sums would not fit the registers;
// one with shares of the keys (decoding).
template <typename T, bool PAGED>
static int launch_attn(const float* q_lat, const void* kc, const void* k_pages, const int* page_table, int table_stride,
                       int ring_pages, const float* sink, void* o_lat, float* part_acc, float* part_ml, int n_splits,
                       int rows_per_block, const int* token_pos, const int* token_seq, const int* cu_seqlens,
                       const int* seq_slot, int row0, int rows, int H, int R, int D, float scale, int window,
                       cudaStream_t stream) {
    const int nc = (R + kAttnThreads - 1) / kAttnThreads;
#define HOS_AS(NC, QT) return launch_attn_as<T, PAGED, NC, QT>(q_lat, kc, k_pages, page_table, table_stride, ring_pages, sink, \
                                                               o_lat, part_acc, part_ml, n_splits, token_pos, token_seq,     \
                                                               cu_seqlens, seq_slot, row0, rows, H, R, D, scale, window, stream)
    if (rows_per_block <= 1 || n_splits > 1) {
        if (nc == 1) HOS_AS(1, 1);
        if (nc == 2) HOS_AS(2, 1);
        HOS_AS(4, 1);
    }
    if (nc == 1) HOS_AS(1, 4);
    if (nc == 2) HOS_AS(2, 2);
    HOS_AS(4, 1);
#undef HOS_AS
}

}  // namespace hos

using namespace hos;

extern "C" const char* hos_last_error() { return error_buffer(); }

extern "C" int hos_latent_prep(const void* proj, int dtype, int proj_stride, int H, int dq, int R, int P,
                               const float* w_norm, float eps, const float* inv_freq, int rot_dims,
                               const int* token_pos, const int* token_seq, const int* seq_slot,
                               const int* seq_len_after, void* kc, float* q_lat, void* k_pages,
                               const int* page_table, int table_stride, int ring_pages, int N, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (rot_dims < 0 || rot_dims > P || (rot_dims & 1)) HOS_REFUSE("latent_prep: %d rotated of %d numbers", rot_dims, P);
    if (dtype == kBF16)
        return launch_prep<bf16>(proj, proj_stride, H, dq, R, P, w_norm, eps, inv_freq, rot_dims, token_pos, token_seq,
                                 seq_slot, seq_len_after, kc, q_lat, k_pages, page_table, table_stride, ring_pages, N, stream);
    if (dtype == kF32)
        return launch_prep<float>(proj, proj_stride, H, dq, R, P, w_norm, eps, inv_freq, rot_dims, token_pos, token_seq,
                                  seq_slot, seq_len_after, kc, q_lat, k_pages, page_table, table_stride, ring_pages, N, stream);
    HOS_REFUSE("latent_prep: unknown dtype %d", dtype);
}

// Rows row0 .. row0 + rows - 1 of the step.  paged = 0: keys are the step's own rows `kc` (sequences
// that start at position 0); paged = 1: keys from `k_pages` through the page table.  n_splits > 1: the keys of
// every row are cut into that many shares (part_acc: [rows of the step][H][n_splits][R], part_ml: [..][n_splits][2]).
// rows_per_block: 1, or more where neighbouring rows share their keys (prompts).  use_tensor_cores: bfloat16 rows
// whose sizes fit take the MMA kernel (the 32-bit query and weights as two bfloat16 terms each); 0 keeps the FMA kernel.
extern "C" int hos_latent_attn(int dtype, int paged, const float* q_lat, const void* kc, const void* k_pages,
                               const int* page_table, int table_stride, int ring_pages, const float* sink,
                               void* o_lat, float* part_acc, float* part_ml, int n_splits, int rows_per_block,
                               const int* token_pos, const int* token_seq, const int* cu_seqlens,
                               const int* seq_slot, int row0, int rows, int H, int R, int D, float scale, int window,
                               int use_tensor_cores, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (R > 4 * kAttnThreads) HOS_REFUSE("latent_attn: a latent of %d numbers is more than %d", R, 4 * kAttnThreads);
    if (R > D) HOS_REFUSE("latent_attn: the latent (%d) is longer than the row (%d)", R, D);
    if (n_splits < 1 || n_splits > 65535 || (n_splits > 1 && (part_acc == nullptr || part_ml == nullptr)))
        HOS_REFUSE("latent_attn: %d shares of the keys need their buffers", n_splits);
#define HOS_GO(T, PG) return launch_attn<T, PG>(q_lat, kc, k_pages, page_table, table_stride, ring_pages, sink, o_lat, part_acc, \
                                                 part_ml, n_splits, rows_per_block, token_pos, token_seq, cu_seqlens, seq_slot,   \
                                                 row0, rows, H, R, D, scale, window, stream)
    if (dtype == kBF16 && use_tensor_cores) {
        const int rc = paged ? launch_attn_tc<true>(q_lat, kc, k_pages, page_table, table_stride, ring_pages, sink, o_lat, part_acc,
                                                    part_ml, n_splits, rows_per_block, token_pos, token_seq, cu_seqlens,
                                                    seq_slot, row0, rows, H, R, D, scale, window, stream)
                             : launch_attn_tc<false>(q_lat, kc, k_pages, page_table, table_stride, ring_pages, sink, o_lat, part_acc,
                                                     part_ml, n_splits, rows_per_block, token_pos, token_seq, cu_seqlens,
                                                     seq_slot, row0, rows, H, R, D, scale, window, stream);
        if (rc <= 0) return rc;
    }
    if (dtype == kBF16 && paged) HOS_GO(bf16, true);
    if (dtype == kBF16) HOS_GO(bf16, false);
    if (dtype == kF32 && paged) HOS_GO(float, true);
    if (dtype == kF32) HOS_GO(float, false);
#undef HOS_GO
    HOS_REFUSE("latent_attn: unknown dtype %d", dtype);
}

// out[m, h, 0:N] = W[h] (N x K, rows contiguous) . in[m, h, 0:K]; strides in elements.
extern "C" int hos_heads_product(const void* in, int in_dtype, const void* W, int w_dtype, void* out, int out_dtype,
                                 int M, int N, int K, int heads, int lda, int a_head, int ldo, int o_head,
                                 cudaStream_t stream) {
    if (M <= 0 || N <= 0 || heads <= 0) return 0;
    if (K <= 0) HOS_REFUSE("heads_product: K must be positive");
    dim3 grid((N + 63) / 64, (M + 63) / 64, heads);
    if (grid.y > 65535 || grid.z > 65535) HOS_REFUSE("heads_product: too many rows or heads for one launch");
    if (in_dtype == kBF16 && w_dtype == kBF16 && K % 8 == 0 && lda % 8 == 0 && a_head % 8 == 0 &&
        ((uintptr_t)in | (uintptr_t)W) % 16 == 0) {
        static bool set = false;
        if (!set) {
            cudaFuncSetAttribute(heads_product_tc_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, TcTile<1>::kSmemBytes);
            cudaFuncSetAttribute(heads_product_tc_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, TcTile<1>::kSmemBytes);
            set = true;
        }
        if (out_dtype == kF32)
            launch_pdl(heads_product_tc_kernel<float>, grid, dim3(256), (size_t)TcTile<1>::kSmemBytes, stream, (const bf16*)in,
                       (const bf16*)W, (float*)out, M, N, K, lda, a_head, ldo, o_head);
        else
            launch_pdl(heads_product_tc_kernel<bf16>, grid, dim3(256), (size_t)TcTile<1>::kSmemBytes, stream, (const bf16*)in,
                       (const bf16*)W, (bf16*)out, M, N, K, lda, a_head, ldo, o_head);
        return check_launch("heads_product");
    }
#define HOS_CASE(da, dw, dout, TA, TW, TO)                                                            \
    if (in_dtype == da && w_dtype == dw && out_dtype == dout) {                                       \
        launch_pdl(heads_product_kernel<TA, TW, TO>, grid, dim3(256), 0, stream, (const TA*)in,       \
                   (const TW*)W, (TO*)out, M, N, K, lda, a_head, N * K, ldo, o_head);                 \
        return check_launch("heads_product");                                                         \
    }
    HOS_CASE(kF32, kF32, kF32, float, float, float)
    HOS_CASE(kBF16, kBF16, kF32, bf16, bf16, float)
    HOS_CASE(kF32, kBF16, kBF16, float, bf16, bf16)
    HOS_CASE(kF32, kBF16, kF32, float, bf16, float)
    HOS_CASE(kBF16, kBF16, kBF16, bf16, bf16, bf16)
#undef HOS_CASE
    HOS_REFUSE("heads_product: no kernel for dtypes in=%d W=%d out=%d", in_dtype, w_dtype, out_dtype);
}
