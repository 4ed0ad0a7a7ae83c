// Softmax attention whose keys and values may differ in size, with query/key norms (per head, or over the whole
// projection), a partial rotation with scaled frequencies, a mask of chunks or of a window (which may keep a
// sequence's first keys in sight), a sink in the denominator and a gate per head.  Everything between the
// projections and the output projection is 32-bit arithmetic.
//
// qk_prep: one block per token over the fused projection row [q | k | v | gate logits] (32-bit, biases added
//   here): each query and key head is divided by its root mean square and multiplied by a weight shared by
//   the heads (norm_whole: the root mean square is taken over all query heads, and over all key heads, at once,
//   and the weight has a number per column), its first rot_dims numbers are rotated as neighbouring pairs
//   (2i, 2i+1) by the angle position * freq[i], cosine and sine times `magnitude`; queries are written as 32-bit
//   rows, keys and values (in the cache's type) to their places in the paged cache.  With v_first the values
//   are first blended with another layer's values of the same token, v <- (1 - v_mix) v + v_mix v_first, and the
//   blend is what the cache holds.
// gated_attn: one warp per (token, up to 8 query heads that share a kv head, share of the keys).  A lane takes a
//   key: 32 scores per head at a time, then the lanes turn to the value columns; a key or value row is read once
//   for all of the warp's heads.  Keys j of position i: j <= i and, with chunks of size C,
//   floor(j / C) = floor(i / C); with a window W, j > i - W or j < keep_first.  The denominator also holds exp(sink[head]).
//   The head's output is multiplied by the logistic function of its gate logit.  With more than one share the
//   partial (maximum, sum, weighted values) go to a workspace and attn_merge adds them.
#include "common.cuh"
#include "kv_layout.cuh"

namespace hos {

struct PagedKV2 {            // keys [n_pages][n_kv][64][kd], values [n_pages][n_kv][64][vd]
    void* k_pages;
    void* v_pages;
    const int* page_table;
    int table_stride;
    int ring_pages;
    int n_kv_heads;
    int kd, vd;
};

__device__ __forceinline__ int table_entry(const PagedKV2& c, int lp) { return c.ring_pages > 0 ? lp % c.ring_pages : lp; }

constexpr int kPrepMaxPL = 16;    // a head of up to 32 * 16 numbers in a warp's registers

template <typename TC, int kPrepPL, int kThreads>
__global__ void __launch_bounds__(kThreads)
qk_prep_kernel(const float* __restrict__ proj, int ld, const float* __restrict__ bias, const float* __restrict__ q_norm,
               const float* __restrict__ k_norm, float eps, const float* __restrict__ freq, int rot_dims, float magnitude,
               const int* __restrict__ token_pos, const int* __restrict__ token_seq, const int* __restrict__ seq_slot,
               float* __restrict__ q_out, PagedKV2 cache, int H, int G, int kd, int vd, int norm_whole,
               const float* __restrict__ v_first, long long v_first_ld, float v_mix, int q_maps) {
    pdl_enter();
    __shared__ float scratch[32];
    const int n = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int seq = token_seq[n];
    const float* row = proj + (size_t)n * ld;
    if (seq < 0) {
        for (int i = threadIdx.x; i < H * kd * q_maps; i += blockDim.x) q_out[(size_t)n * H * kd * q_maps + i] = 0.f;
        return;
    }
    const int pos = token_pos[n];
    const float fpos = (float)pos;
    const int slot = seq_slot[seq];
    const int page = G > 0 ? cache.page_table[(size_t)slot * cache.table_stride + table_entry(cache, pos / kPageTokens)] : 0;
    const int r = pos % kPageTokens;
    float inv_all[2] = {0.f, 0.f};                       // norm_whole: one root mean square for all q heads, one for all k heads
    if (norm_whole) {
        for (int part = 0; part < (G > 0 ? 2 : 1); ++part) {
            const int c0 = part == 0 ? 0 : H * kd, cn = part == 0 ? H * kd : G * kd;
            float ss = 0.f;
            for (int i = threadIdx.x; i < cn; i += blockDim.x) {
                const float x = row[c0 + i] + (bias ? bias[c0 + i] : 0.f);
                ss = fmaf(x, x, ss);
            }
            ss = block_sum(ss, scratch);
            inv_all[part] = 1.f / sqrtf(ss / (float)cn + eps);
        }
    }
    // query heads 0..H-1, then key heads H..H+G-1
    for (int item = warp; item < H + G; item += kThreads / 32) {
        const bool is_q = item < H;
        const int col0 = item * kd;                      // q heads and k heads follow one another in the row
        const float* nw = is_q ? q_norm : k_norm;
        if (nw != nullptr && norm_whole) nw += (is_q ? item : item - H) * kd;
        float v[kPrepPL];
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < kPrepPL; ++i) {
            const int d = lane + 32 * i;
            v[i] = d < kd ? row[col0 + d] + (bias ? bias[col0 + d] : 0.f) : 0.f;
            ss = fmaf(v[i], v[i], ss);
        }
        if (nw != nullptr) {
            ss = warp_sum(ss);
            const float inv = norm_whole ? inv_all[is_q ? 0 : 1] : 1.f / sqrtf(ss / (float)kd + eps);
#pragma unroll
            for (int i = 0; i < kPrepPL; ++i) {
                const int d = lane + 32 * i;
                if (d < kd) v[i] = v[i] * inv * nw[d];
            }
        }
#pragma unroll
        for (int i = 0; i < kPrepPL; ++i) {
            const int d = lane + 32 * i;
            const float other = __shfl_xor_sync(0xffffffffu, v[i], 1);       // the pair's partner: the lane beside
            if (d < rot_dims && d < kd) {
                float sn, cs;
                sincosf(fpos * freq[d >> 1], &sn, &cs);
                sn *= magnitude;
                cs *= magnitude;
                v[i] = (d & 1) ? fmaf(v[i], cs, other * sn) : fmaf(v[i], cs, -other * sn);
            }
        }
        if (is_q && q_maps > 1) {
            // a head's kd numbers are q_maps queries of kd / q_maps numbers each, one per attention map over the same
            // key row: query m is written as a head of its own, zero outside its own part of the key row
            const int md = kd / q_maps;
            float* qo = q_out + ((size_t)n * H + item) * q_maps * kd;
            for (int m = 0; m < q_maps; ++m)
#pragma unroll
                for (int i = 0; i < kPrepPL; ++i) {
                    const int d = lane + 32 * i;
                    if (d < kd) qo[(size_t)m * kd + d] = d / md == m ? v[i] : 0.f;
                }
        } else if (is_q) {
            float* qo = q_out + ((size_t)n * H + item) * kd;
#pragma unroll
            for (int i = 0; i < kPrepPL; ++i) {
                const int d = lane + 32 * i;
                if (d < kd) qo[d] = v[i];
            }
        } else {
            const int g = item - H;
            TC* kp = (TC*)cache.k_pages + ((size_t)page * G + g) * (size_t)kPageTokens * kd;
#pragma unroll
            for (int i = 0; i < kPrepPL; ++i) {
                const int d = lane + 32 * i;
                if (d < kd) kp[kv_elem_offset(r, d, kd)] = from_float<TC>(v[i]);
            }
        }
    }
    if (G > 0) {
        const int col0 = (H + G) * kd;
        for (int i = threadIdx.x; i < G * vd; i += blockDim.x) {
            const int g = i / vd, d = i % vd;
            TC* vp = (TC*)cache.v_pages + ((size_t)page * G + g) * (size_t)kPageTokens * vd;
            float x = row[col0 + i] + (bias ? bias[col0 + i] : 0.f);
            if (v_first != nullptr) x = fmaf(v_mix, v_first[(size_t)n * v_first_ld + i], (1.f - v_mix) * x);
            vp[kv_elem_offset(r, d, vd)] = from_float<TC>(x);
        }
    }
}

constexpr int kAttnWarps = 4;
constexpr int kMaxVPL = 16;       // value heads of up to 32 * 16 numbers

// 8 numbers of a cache row, whatever the type
__device__ __forceinline__ void load8(const float* p, float (&f)[8]) {
    const float4 a = *(const float4*)p, b = *(const float4*)(p + 4);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
__device__ __forceinline__ void load8(const bf16* p, float (&f)[8]) {
    const uint4 u = *(const uint4*)p;
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

template <typename TC, int VPL, int QH>
__global__ void __launch_bounds__(kAttnWarps * 32)
gated_attn_kernel(const float* __restrict__ q, PagedKV2 cache, const float* __restrict__ sink, const float* __restrict__ gate,
                  long long gate_stride, const int* __restrict__ token_pos, const int* __restrict__ token_seq,
                  const int* __restrict__ seq_slot, void* __restrict__ out, int out_bf16, float* __restrict__ part_acc,
                  float* __restrict__ part_ml, int n_splits, int n_tokens, int H, int G, int kd, int vd, float scale,
                  int chunk, int window, int keep_first) {
    pdl_enter();
    extern __shared__ float qs_all[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int groups = H / QH;                       // QH query heads that share a kv head go together: its keys and
    const long long item = (long long)blockIdx.x * kAttnWarps + warp;      // values are read once for all of them
    if (item >= (long long)n_tokens * groups * n_splits) return;
    const int split = (int)(item % n_splits);
    const int h0 = (int)((item / n_splits) % groups) * QH, n = (int)(item / ((long long)n_splits * groups));
    const int seq = token_seq[n];
    if (seq < 0) {
#pragma unroll
        for (int hh = 0; hh < QH; ++hh) {
            const size_t orow = ((size_t)n * H + h0 + hh) * vd;
            if (n_splits == 1)
                for (int d = lane; d < vd; d += 32) {
                    if (out_bf16) ((bf16*)out)[orow + d] = from_float<bf16>(0.f);
                    else ((float*)out)[orow + d] = 0.f;
                }
            else if (lane < 2)
                part_ml[(((size_t)n * H + h0 + hh) * n_splits + split) * 2 + lane] = lane == 0 ? -INFINITY : 0.f;
        }
        return;
    }
    const int pos = token_pos[n];
    const int g = h0 / (H / G);
    int first = 0;
    if (chunk > 0) first = pos / chunk * chunk;
    if (window > 0) first = max(first, pos + 1 - window);
    // the keys a row sees, counted u = 0, 1, ...: the sequence's first `kept` keys (those of the first keep_first that the
    // mask's lower edge has passed), then the keys first .. pos; key_of(u) is the position of the u-th
    const int kept = min(max(keep_first, 0), first), shift = first - kept;
    int lo = 0, hi = kept + pos + 1 - first;
    if (n_splits > 1) {       // shares are runs of whole blocks of 32 keys
        const int blocks = (hi - lo + 31) / 32, per = (blocks + n_splits - 1) / n_splits;
        const int a = lo + split * per * 32;
        hi = min(hi, a + per * 32);
        lo = a;
    }
    float* qs = qs_all + warp * QH * kd;
    const float* qp = q + ((size_t)n * H + h0) * kd;
    for (int d = lane; d < QH * kd; d += 32) qs[d] = qp[d];
    __syncwarp();
    const int slot = seq_slot[seq];
    const int* table = cache.page_table + (size_t)slot * cache.table_stride;

    // the sink takes part once: in the first share
    const bool with_sink = sink != nullptr && split == 0;
    float m[QH], l[QH], acc[QH][VPL];
#pragma unroll
    for (int hh = 0; hh < QH; ++hh) {
        m[hh] = with_sink ? sink[h0 + hh] : -INFINITY;
        l[hh] = with_sink ? 1.f : 0.f;
#pragma unroll
        for (int i = 0; i < VPL; ++i) acc[hh][i] = 0.f;
    }
    const bool vec = (kd & 7) == 0;

    for (int t0 = lo; t0 < hi; t0 += 32) {
        const int u = t0 + lane, t = u < kept ? u : u + shift;
        float s[QH];
#pragma unroll
        for (int hh = 0; hh < QH; ++hh) s[hh] = -INFINITY;
        int my_page = 0;
        if (u < hi) {
            my_page = table[table_entry(cache, t / kPageTokens)];
            const int r = t % kPageTokens;
            const TC* kp = (const TC*)cache.k_pages + ((size_t)my_page * G + g) * (size_t)kPageTokens * kd;
            float dot[QH];
#pragma unroll
            for (int hh = 0; hh < QH; ++hh) dot[hh] = 0.f;
            if (vec) {
                for (int c = 0; c < kd; c += 8) {
                    float f[8];
                    load8(kp + kv_elem_offset(r, c, kd), f);
#pragma unroll
                    for (int hh = 0; hh < QH; ++hh)
#pragma unroll
                        for (int e = 0; e < 8; ++e) dot[hh] = fmaf(qs[hh * kd + c + e], f[e], dot[hh]);
                }
            } else {
                for (int d = 0; d < kd; ++d) {
                    const float kv = to_float(kp[kv_elem_offset(r, d, kd)]);
#pragma unroll
                    for (int hh = 0; hh < QH; ++hh) dot[hh] = fmaf(qs[hh * kd + d], kv, dot[hh]);
                }
            }
#pragma unroll
            for (int hh = 0; hh < QH; ++hh) s[hh] = dot[hh] * scale;
        }
        float p[QH];
#pragma unroll
        for (int hh = 0; hh < QH; ++hh) {
            const float m_new = fmaxf(m[hh], warp_max(s[hh]));
            const float corr = expf(m[hh] - m_new);          // m_new is finite here: the block holds one key at least
            p[hh] = u < hi ? expf(s[hh] - m_new) : 0.f;
            l[hh] = l[hh] * corr + warp_sum(p[hh]);
#pragma unroll
            for (int i = 0; i < VPL; ++i) acc[hh][i] *= corr;
            m[hh] = m_new;
        }
        const int cnt = min(32, hi - t0);
        for (int j = 0; j < cnt; ++j) {
            const int pg = __shfl_sync(0xffffffffu, my_page, j);
            const int r = (t0 + j < kept ? t0 + j : t0 + j + shift) % kPageTokens;
            const TC* vp = (const TC*)cache.v_pages + ((size_t)pg * G + g) * (size_t)kPageTokens * vd;
            float vv[VPL];
#pragma unroll
            for (int i = 0; i < VPL; ++i) {
                const int d = lane + 32 * i;
                vv[i] = d < vd ? to_float(vp[kv_elem_offset(r, d, vd)]) : 0.f;
            }
#pragma unroll
            for (int hh = 0; hh < QH; ++hh) {
                const float pj = __shfl_sync(0xffffffffu, p[hh], j);
#pragma unroll
                for (int i = 0; i < VPL; ++i) acc[hh][i] = fmaf(pj, vv[i], acc[hh][i]);
            }
        }
    }
#pragma unroll
    for (int hh = 0; hh < QH; ++hh) {
        const int h = h0 + hh;
        const size_t orow = ((size_t)n * H + h) * vd;
        if (n_splits > 1) {
            const size_t pi = ((size_t)n * H + h) * n_splits + split;
            if (lane == 0) {
                part_ml[pi * 2] = m[hh];
                part_ml[pi * 2 + 1] = l[hh];
            }
#pragma unroll
            for (int i = 0; i < VPL; ++i) {
                const int d = lane + 32 * i;
                if (d < vd) part_acc[pi * vd + d] = acc[hh][i];
            }
            continue;
        }
        float f = l[hh] > 0.f ? 1.f / l[hh] : 0.f;
        if (gate != nullptr) f *= 1.f / (1.f + expf(-gate[(size_t)n * gate_stride + h]));
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            const int d = lane + 32 * i;
            if (d < vd) {
                if (out_bf16) ((bf16*)out)[orow + d] = from_float<bf16>(acc[hh][i] * f);
                else ((float*)out)[orow + d] = acc[hh][i] * f;
            }
        }
    }
}

// one warp per (token, head): the shares' sums under one maximum.  The lanes first take a share each (maximum and
// sum), then 128 value columns at a time, four to a lane, with the shares' rows as independent loads.
__global__ void __launch_bounds__(128)
attn_merge_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml, int n_splits,
                  const float* __restrict__ gate, long long gate_stride, const int* __restrict__ token_seq,
                  void* __restrict__ out, int out_bf16, int n_tokens, int H, int vd) {
    pdl_enter();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * 4 + warp;
    if (item >= (long long)n_tokens * H) return;
    const int n = (int)(item / H), h = (int)(item % H);
    const float* ml = part_ml + (size_t)item * n_splits * 2;
    const bool live = token_seq[n] >= 0;
    float m = -INFINITY;
    if (live)
        for (int s = lane; s < n_splits; s += 32) m = fmaxf(m, ml[2 * s]);
    m = warp_max(m);
    float l = 0.f;
    if (live)
        for (int s = lane; s < n_splits; s += 32) l += ml[2 * s + 1] > 0.f ? ml[2 * s + 1] * expf(ml[2 * s] - m) : 0.f;
    l = warp_sum(l);
    float f = l > 0.f ? 1.f / l : 0.f;
    if (live && gate != nullptr) f *= 1.f / (1.f + expf(-gate[(size_t)n * gate_stride + h]));
    const float* acc_rows = part_acc + (size_t)item * n_splits * vd;
    for (int d0 = 0; d0 < vd; d0 += 128) {
        float a[4] = {0.f, 0.f, 0.f, 0.f};
        if (live) {
#pragma unroll 4
            for (int s = 0; s < n_splits; ++s) {
                const float w = ml[2 * s + 1] > 0.f ? expf(ml[2 * s] - m) : 0.f;     // a share without keys: its row does not count
                float x[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int d = d0 + lane + 32 * i;
                    x[i] = d < vd ? acc_rows[(size_t)s * vd + d] : 0.f;
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) a[i] = w > 0.f ? fmaf(x[i], w, a[i]) : a[i];
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int d = d0 + lane + 32 * i;
            if (d >= vd) continue;
            if (out_bf16) ((bf16*)out)[(size_t)item * vd + d] = from_float<bf16>(a[i] * f);
            else ((float*)out)[(size_t)item * vd + d] = a[i] * f;
        }
    }
}

// Two attention maps over the same values, combined: a [N][H][2][vd] float32 (map 1 and map 2 of a head side by side);
// out[n][h][:] = rms_norm(a1 - lambda a2) * mult * logistic(gate[n][h * vd + :]); the root mean square is per head
// (eps inside the root, no weight).  A warp per (token, head).
template <typename TO>
__global__ void __launch_bounds__(128)
diff_combine_kernel(const float* __restrict__ a, float lambda, float mult, float eps, const float* __restrict__ gate,
                    long long gate_stride, const int* __restrict__ token_seq, TO* __restrict__ out, int N, int H, int vd) {
    pdl_enter();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * 4 + warp;
    if (item >= (long long)N * H) return;
    const int n = (int)(item / H), h = (int)(item % H);
    TO* op = out + (size_t)item * vd;
    if (token_seq[n] < 0) {
        for (int d = lane; d < vd; d += 32) op[d] = from_float<TO>(0.f);
        return;
    }
    const float* a1 = a + (size_t)item * 2 * vd;
    const float* a2 = a1 + vd;
    float ss = 0.f;
    for (int d = lane; d < vd; d += 32) {
        const float o = fmaf(-lambda, a2[d], a1[d]);
        ss = fmaf(o, o, ss);
    }
    ss = warp_sum(ss);
    const float f = mult / sqrtf(ss / (float)vd + eps);
    const float* gt = gate != nullptr ? gate + (size_t)n * gate_stride + (size_t)h * vd : nullptr;
    for (int d = lane; d < vd; d += 32) {
        float o = fmaf(-lambda, a2[d], a1[d]) * f;
        if (gt != nullptr) o *= 1.f / (1.f + expf(-gt[d]));
        op[d] = from_float<TO>(o);
    }
}

}  // namespace hos

using namespace hos;

extern "C" const char* hos_last_error() { return error_buffer(); }

// proj: float32 [N][ld], columns q (H * kd), then k (G * kd) and v (G * vd) if G > 0 (a call that reads another
// call's cache passes G = 0 and projects neither), then whatever else the caller keeps there.  bias: the same
// columns' biases or null.  q_norm / k_norm: [kd] or null (norm_whole: [H * kd] and [G * kd]).  freq: [rot_dims / 2] or
// null.  v_first: row n's values of another layer at v_first[n * v_first_ld + ...] (G * vd numbers), or null.
// q_maps > 1: q_out is [N][H * q_maps][kd]: each head's kd numbers are q_maps queries, written as heads of their own.
extern "C" int hos_qk_prep(const float* proj, int ld, const float* bias, const float* q_norm, const float* k_norm, float eps,
                           const float* freq, int rot_dims, float magnitude, const int* token_pos, const int* token_seq,
                           const int* seq_slot, float* q_out, void* k_pages, void* v_pages, int cache_dtype,
                           const int* page_table, int table_stride, int ring_pages, int N, int H, int G, int kd, int vd,
                           int norm_whole, const float* v_first, long long v_first_ld, float v_mix, int q_maps,
                           cudaStream_t stream) {
    if (N <= 0) return 0;
    if (q_maps < 1 || kd % q_maps != 0) HOS_REFUSE("qk_prep: heads of %d numbers do not hold %d queries", kd, q_maps);
    if (kd <= 0 || kd > 32 * kPrepMaxPL) HOS_REFUSE("qk_prep: heads of %d numbers are outside 1..%d", kd, 32 * kPrepMaxPL);
    if (freq == nullptr) rot_dims = 0;
    if (rot_dims % 2 != 0 || rot_dims > kd) HOS_REFUSE("qk_prep: %d rotated numbers in heads of %d", rot_dims, kd);
    PagedKV2 c{k_pages, v_pages, page_table, table_stride, ring_pages, G, kd, vd};
    // few rows (single-token steps): a block of 16 warps shortens the row's chain of loads; many rows: 4 warps
    const bool wide = N <= 592 && H + G > 4;
#define HOS_QKP_N(TC, PL, NT)                                                                                        \
    launch_pdl(qk_prep_kernel<TC, PL, NT>, dim3(N), dim3(NT), 0, stream, proj, ld, bias, q_norm, k_norm, eps, freq,   \
               rot_dims, magnitude, token_pos, token_seq, seq_slot, q_out, c, H, G, kd, vd, norm_whole, v_first,     \
               v_first_ld, v_mix, q_maps)
#define HOS_QKP(TC, PL)                                                                                              \
    do {                                                                                                             \
        if (wide) HOS_QKP_N(TC, PL, 512);                                                                            \
        else HOS_QKP_N(TC, PL, 128);                                                                                 \
    } while (0)
#define HOS_QKP_T(TC)                                                                                                \
    do {                                                                                                             \
        if (kd <= 32) HOS_QKP(TC, 1);                                                                                \
        else if (kd <= 64) HOS_QKP(TC, 2);                                                                           \
        else if (kd <= 128) HOS_QKP(TC, 4);                                                                          \
        else if (kd <= 256) HOS_QKP(TC, 8);                                                                          \
        else HOS_QKP(TC, 16);                                                                                        \
    } while (0)
    if (cache_dtype == kBF16) HOS_QKP_T(bf16);
    else HOS_QKP_T(float);
#undef HOS_QKP_T
#undef HOS_QKP
#undef HOS_QKP_N
    return check_launch("qk_prep");
}

// q: float32 [N][H][kd].  out: [N][H][vd] of out_dtype.  gate: row n's logit of head h at gate[n * gate_stride + h], or
// null.  sink: [H] or null.  chunk, window: 0 for none; keep_first: with a window, that many of a sequence's first keys
// stay in sight.  n_splits > 1: part_acc [N][H][n_splits][vd] and part_ml
// [N][H][n_splits][2] float32 must be given.
extern "C" int hos_gated_attn(const float* q, void* k_pages, void* v_pages, int cache_dtype, const int* page_table,
                              int table_stride, int ring_pages, const float* sink, const float* gate, long long gate_stride,
                              const int* token_pos, const int* token_seq, const int* seq_slot, void* out, int out_dtype,
                              float* part_acc, float* part_ml, int n_splits, int N, int H, int G, int kd, int vd, float scale,
                              int chunk, int window, int keep_first, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (G <= 0 || H % G != 0) HOS_REFUSE("gated_attn: %d heads are not a multiple of %d kv heads", H, G);
    if (vd <= 0 || vd > 32 * kMaxVPL) HOS_REFUSE("gated_attn: value heads of %d numbers are outside 1..%d", vd, 32 * kMaxVPL);
    if (n_splits < 1 || (n_splits > 1 && (part_acc == nullptr || part_ml == nullptr)))
        HOS_REFUSE("gated_attn: %d shares need a workspace", n_splits);
    // query heads that share a kv head go to one warp, as many as its registers and shared memory take
    const int vpl = vd <= 32 ? 1 : (vd <= 64 ? 2 : (vd <= 128 ? 4 : (vd <= 256 ? 8 : 16)));
    int qh = 1;
    for (int c = 8; c > 1; c >>= 1)
        if ((H / G) % c == 0 && c * vpl <= 32 && (size_t)kAttnWarps * c * kd * sizeof(float) <= 48 * 1024) {
            qh = c;
            break;
        }
    const size_t smem = (size_t)kAttnWarps * qh * kd * sizeof(float);
    if (smem > 48 * 1024) HOS_REFUSE("gated_attn: heads of %d numbers do not fit", kd);
    PagedKV2 c{k_pages, v_pages, page_table, table_stride, ring_pages, G, kd, vd};
    const long long items = (long long)N * (H / qh) * n_splits;
    const unsigned blocks = (unsigned)((items + kAttnWarps - 1) / kAttnWarps);
    const int out_bf16 = out_dtype == kBF16;
#define HOS_GA(TC, VPL, QH)                                                                                          \
    launch_pdl(gated_attn_kernel<TC, VPL, QH>, dim3(blocks), dim3(kAttnWarps * 32), smem, stream, q, c, sink, gate,  \
               gate_stride, token_pos, token_seq, seq_slot, out, out_bf16, part_acc, part_ml, n_splits, N, H, G, kd, vd, \
               scale, chunk, window, keep_first)
#define HOS_GA_Q(TC, VPL)                                                                                            \
    do {                                                                                                             \
        if (qh == 8) { if constexpr (VPL <= 4) HOS_GA(TC, VPL, 8); }                                                 \
        else if (qh == 4) { if constexpr (VPL <= 8) HOS_GA(TC, VPL, 4); }                                            \
        else if (qh == 2) HOS_GA(TC, VPL, 2);                                                                        \
        else HOS_GA(TC, VPL, 1);                                                                                     \
    } while (0)
#define HOS_GA_T(TC)                                                                                                 \
    do {                                                                                                             \
        if (vd <= 32) HOS_GA_Q(TC, 1);                                                                               \
        else if (vd <= 64) HOS_GA_Q(TC, 2);                                                                          \
        else if (vd <= 128) HOS_GA_Q(TC, 4);                                                                         \
        else if (vd <= 256) HOS_GA_Q(TC, 8);                                                                         \
        else HOS_GA_Q(TC, 16);                                                                                       \
    } while (0)
    if (cache_dtype == kBF16) HOS_GA_T(bf16);
    else HOS_GA_T(float);
#undef HOS_GA_T
#undef HOS_GA_Q
#undef HOS_GA
    int rc = check_launch("gated_attn");
    if (rc != 0 || n_splits == 1) return rc;
    launch_pdl(attn_merge_kernel, dim3((unsigned)(((long long)N * H + 3) / 4)), dim3(128), 0, stream, (const float*)part_acc,
               (const float*)part_ml, n_splits, gate, gate_stride, token_seq, out, out_bf16, N, H, vd);
    return check_launch("attn_merge");
}

// The shares' partial results under one maximum: out [N][H][vd] from part_acc [N][H][n_splits][vd], part_ml [..][2].
extern "C" int hos_attn_merge(const float* part_acc, const float* part_ml, int n_splits, const float* gate,
                              long long gate_stride, const int* token_seq, void* out, int out_dtype, int N, int H, int vd,
                              cudaStream_t stream) {
    if (N <= 0) return 0;
    launch_pdl(attn_merge_kernel, dim3((unsigned)(((long long)N * H + 3) / 4)), dim3(128), 0, stream, part_acc, part_ml,
               n_splits, gate, gate_stride, token_seq, out, out_dtype == kBF16 ? 1 : 0, N, H, vd);
    return check_launch("attn_merge");
}

// a: float32 [N][H][2][vd], the two maps' outputs of every head; out: [N][H][vd] of out_dtype; gate: row n's logits for
// the H * vd output columns at gate[n * gate_stride + ...], or null.
extern "C" int hos_diff_combine(const float* a, float lambda, float mult, float eps, const float* gate, long long gate_stride,
                                const int* token_seq, void* out, int out_dtype, int N, int H, int vd, cudaStream_t stream) {
    if (N <= 0) return 0;
    const unsigned blocks = (unsigned)(((long long)N * H + 3) / 4);
    if (out_dtype == kBF16)
        launch_pdl(diff_combine_kernel<bf16>, dim3(blocks), dim3(128), 0, stream, a, lambda, mult, eps, gate, gate_stride,
                   token_seq, (bf16*)out, N, H, vd);
    else if (out_dtype == kF32)
        launch_pdl(diff_combine_kernel<float>, dim3(blocks), dim3(128), 0, stream, a, lambda, mult, eps, gate, gate_stride,
                   token_seq, (float*)out, N, H, vd);
    else
        HOS_REFUSE("diff_combine: unknown dtype %d", out_dtype);
    return check_launch("diff_combine");
}
