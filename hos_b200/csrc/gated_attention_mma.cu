// The attention of gated_attention.cu for rows that come many to a sequence (prompts, pieces of prompts), in
// bfloat16 on the tensor cores, flash style, over the paged cache.
//
// One CTA (4 warps) takes 64 consecutive rows of one sequence and one query head; key and value tiles of 64
// positions are pages of the cache, copied as they lie (the cache's permutation of 16-byte groups is the one the
// kernel reads with) through a two-stage cp.async pipeline.  Per tile each warp computes S = Q K^T for its 16
// queries (m16n8k16, 32-bit accumulators: with bfloat16 operands every product is exact, so the scores are 32-bit
// sums), scales, masks (causal; the chunk's first key; the window's edge, with or without a sequence's kept first keys), keeps the running maximum and sum in
// 32-bit and accumulates O += P V with the 32-bit weights P fed as two bfloat16 terms (P = hi + lo, 16 bits of
// mantissa) so that the weights are not rounded to 8 bits.  The sink starts the running maximum and the sum
// (exp(sink - max) counts once); the head's gate multiplies the output.  Keys of KD and values of VD numbers,
// compiled for 64 and 128 each.
#include "common.cuh"
#include "kv_layout.cuh"
#include "mma_utils.cuh"

namespace hos {

constexpr int MQ = 64, MK = 64;       // queries per CTA, keys per tile (a page)

__device__ __forceinline__ void cp16(void* smem_dst, const void* gmem_src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int KD, int VD>
__global__ void __launch_bounds__(128)
gated_attn_mma_kernel(const float* __restrict__ q, const bf16* __restrict__ k_pages, const bf16* __restrict__ v_pages,
                      const int* __restrict__ page_table, int table_stride, int ring_pages, const float* __restrict__ sink,
                      const float* __restrict__ gate, long long gate_stride, const int* __restrict__ cu_seqlens,
                      const int* __restrict__ token_pos, const int* __restrict__ token_seq, const int* __restrict__ seq_slot,
                      void* __restrict__ out_v, int out_f32, int n_seqs, int H, int G, float scale, int chunk, int window,
                      int keep_first) {
    pdl_enter();
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* q_s = reinterpret_cast<bf16*>(smem_raw);                 // [64][KD]
    bf16* kv_s = q_s + MQ * KD;                                    // stage s: K [64][KD] then V [64][VD]
    constexpr int kStage = MK * (KD + VD);

    int seq = 0, tile_in_seq = blockIdx.x, row0 = 0, len = 0;
    for (; seq < n_seqs; ++seq) {
        row0 = cu_seqlens[seq];
        len = cu_seqlens[seq + 1] - row0;
        if (len > 0 && token_seq[row0] < 0) len = 0;               // padding
        const int nt = (len + MQ - 1) / MQ;
        if (tile_in_seq < nt) break;
        tile_in_seq -= nt;
    }
    if (seq >= n_seqs) return;
    const int head = blockIdx.y, kvh = head / (H / G);
    const int q0 = tile_in_seq * MQ;
    const int q_rows = min(MQ, len - q0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
    const int p0 = token_pos[row0] + q0;                            // the position of the CTA's first query
    const int last_q = p0 + q_rows - 1;
    int first_key = chunk > 0 ? p0 / chunk * chunk : 0;
    if (window > 0) first_key = max(first_key, p0 + 1 - window);
    const int kt_lo = first_key / MK, kt_hi = last_q / MK;
    // with kept first keys, their tiles come first (those that lie before the mask's own first tile)
    const int n_keep = keep_first > 0 ? min((keep_first + MK - 1) / MK, kt_lo) : 0;
    const int n_kt = n_keep + kt_hi - kt_lo + 1;
    auto tile_of = [&](int it) { return it < n_keep ? it : kt_lo + it - n_keep; };
    const int* table = page_table + (size_t)seq_slot[seq] * table_stride;

    auto load_kv = [&](int kt, int stage) {
        const int lp = kt;                                          // a tile is a page
        const int page = table[ring_pages > 0 ? lp % ring_pages : lp];
        const bf16* ksrc = k_pages + ((size_t)page * G + kvh) * (size_t)kPageTokens * KD;
        const bf16* vsrc = v_pages + ((size_t)page * G + kvh) * (size_t)kPageTokens * VD;
        bf16* ks = kv_s + (size_t)stage * kStage;
        bf16* vs = ks + MK * KD;
        for (int i = threadIdx.x; i < MK * (KD / 8); i += 128) cp16(ks + i * 8, ksrc + i * 8);
        for (int i = threadIdx.x; i < MK * (VD / 8); i += 128) cp16(vs + i * 8, vsrc + i * 8);
    };
    load_kv(tile_of(0), 0);                                         // under way while the queries are staged
    cp_commit();
    // the queries: 32-bit rows, rounded here to the tensor cores' type; rows beyond the sequence are zeros
    for (int i = threadIdx.x; i < MQ * (KD / 8); i += 128) {
        const int r = i / (KD / 8), c = i % (KD / 8);
        uint4 packed = make_uint4(0u, 0u, 0u, 0u);
        if (r < q_rows) {
            const float* src = q + ((size_t)(row0 + q0 + r) * H + head) * KD + c * 8;
            const float4 a = *(const float4*)src, b = *(const float4*)(src + 4);
            packed = make_uint4(pack_bf16(a.x, a.y), pack_bf16(a.z, a.w), pack_bf16(b.x, b.y), pack_bf16(b.z, b.w));
        }
        *reinterpret_cast<uint4*>(q_s + tile_chunk_offset<KD>(r, c)) = packed;
    }

    const float sk = sink != nullptr ? sink[head] : -INFINITY;
    float m_run[2] = {sk, sk};
    float l_run[2] = {(sink != nullptr && t4 == 0) ? 1.f : 0.f, (sink != nullptr && t4 == 0) ? 1.f : 0.f};
    float o[VD / 8][4];
#pragma unroll
    for (int i = 0; i < VD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    const uint32_t q_base = smem_u32(q_s);
    const int qpos[2] = {p0 + warp * 16 + g, p0 + warp * 16 + g + 8};
    int qlo[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        qlo[r] = chunk > 0 ? qpos[r] / chunk * chunk : 0;
        if (window > 0) qlo[r] = max(qlo[r], qpos[r] + 1 - window);
    }
    // the largest first key among the warp's 16 queries (its last one's)
    int qlo_max;
    {
        const int q_last = p0 + warp * 16 + 15;
        qlo_max = chunk > 0 ? q_last / chunk * chunk : 0;
        if (window > 0) qlo_max = max(qlo_max, q_last + 1 - window);
    }

    for (int it = 0; it < n_kt; ++it) {
        const int stage = it & 1;
        if (it + 1 < n_kt) load_kv(tile_of(it + 1), stage ^ 1);
        cp_commit();
        cp_wait<1>();
        __syncthreads();
        const uint32_t k_base = smem_u32(kv_s + (size_t)stage * kStage);
        const uint32_t v_base = k_base + 2 * MK * KD;
        const int key0 = tile_of(it) * MK;

        float sc[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i) sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < KD / 16; ++kk) {
            uint32_t qa[4];
            {
                const int row = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                ldmatrix_x4(qa, q_base + 2 * tile_chunk_offset<KD>(row, kk * 2 + (lane >> 4)));
            }
#pragma unroll
            for (int kb = 0; kb < 4; ++kb) {
                uint32_t b[4];
                const int row = kb * 16 + (lane & 7) + (lane >> 4) * 8;
                ldmatrix_x4(b, k_base + 2 * tile_chunk_offset<KD>(row, kk * 2 + ((lane >> 3) & 1)));
                mma_bf16(sc[kb * 2], qa, b[0], b[1]);
                mma_bf16(sc[kb * 2 + 1], qa, b[2], b[3]);
            }
        }
        float m_new[2] = {m_run[0], m_run[1]};
        // a tile that every query of the warp sees whole (after its first key, up to its own position, or kept) skips the mask
        const bool whole = key0 + MK - 1 <= p0 + warp * 16 && (key0 >= qlo_max || key0 + MK <= keep_first);
        if (whole) {
#pragma unroll
            for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    sc[nt][i] *= scale;
                    m_new[i >> 1] = fmaxf(m_new[i >> 1], sc[nt][i]);
                }
        } else {
#pragma unroll
            for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int key = key0 + nt * 8 + 2 * t4 + (i & 1);
                    const bool vis = key <= qpos[i >> 1] && (key >= qlo[i >> 1] || key < keep_first);
                    const float s = vis ? sc[nt][i] * scale : -INFINITY;
                    sc[nt][i] = s;
                    m_new[i >> 1] = fmaxf(m_new[i >> 1], s);
                }
        }
        float corr[2], m_use[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            m_new[r] = fmaxf(m_new[r], __shfl_xor_sync(0xffffffffu, m_new[r], 1));
            m_new[r] = fmaxf(m_new[r], __shfl_xor_sync(0xffffffffu, m_new[r], 2));
            m_use[r] = m_new[r] == -INFINITY ? 0.f : m_new[r];
            corr[r] = __expf(m_run[r] - m_use[r]);
            m_run[r] = m_new[r];
            l_run[r] *= corr[r];
        }
#pragma unroll
        for (int i = 0; i < VD / 8; ++i) {
            o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1];
        }
#pragma unroll
        for (int kb = 0; kb < 4; ++kb) {
            uint32_t hi[4], lo[4];
            {
                float p[2][4];
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        p[h][i] = __expf(sc[kb * 2 + h][i] - m_use[i >> 1]);
                        l_run[i >> 1] += p[h][i];
                    }
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const float a = p[h][2 * j], b = p[h][2 * j + 1];
                        const uint32_t top = pack_bf16(a, b);        // both rounded in one conversion; the halves widen by shifts
                        hi[h * 2 + j] = top;
                        lo[h * 2 + j] = pack_bf16(a - __uint_as_float(top << 16), b - __uint_as_float(top & 0xffff0000u));
                    }
            }
            // four value blocks at a time: eight accumulators take the high terms, then the low ones, so that an
            // MMA does not wait for the one just issued into the same accumulator
#pragma unroll
            for (int d4 = 0; d4 < VD / 16; d4 += 4) {
                uint32_t vb[4][4];
                const int row = kb * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    ldmatrix_x4_trans(vb[j], v_base + 2 * tile_chunk_offset<VD>(row, (d4 + j) * 2 + (lane >> 4)));
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    mma_bf16(o[(d4 + j) * 2], hi, vb[j][0], vb[j][1]);
                    mma_bf16(o[(d4 + j) * 2 + 1], hi, vb[j][2], vb[j][3]);
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    mma_bf16(o[(d4 + j) * 2], lo, vb[j][0], vb[j][1]);
                    mma_bf16(o[(d4 + j) * 2 + 1], lo, vb[j][2], vb[j][3]);
                }
            }
        }
        __syncthreads();
    }
    cp_wait<0>();
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int qi = warp * 16 + g + r * 8;
        if (qi >= q_rows) continue;
        const size_t row = (size_t)(row0 + q0 + qi);
        float f = l_run[r] > 0.f ? 1.f / l_run[r] : 0.f;
        if (gate != nullptr) f *= 1.f / (1.f + expf(-gate[row * gate_stride + head]));
        if (out_f32) {          // a caller that goes on computing with the heads' outputs takes them unrounded
            float* op = (float*)out_v + (row * H + head) * VD;
#pragma unroll
            for (int i = 0; i < VD / 8; ++i)
                *reinterpret_cast<float2*>(op + i * 8 + 2 * t4) = make_float2(o[i][2 * r] * f, o[i][2 * r + 1] * f);
            continue;
        }
        bf16* op = (bf16*)out_v + (row * H + head) * VD;
#pragma unroll
        for (int i = 0; i < VD / 8; ++i)
            *reinterpret_cast<uint32_t*>(op + i * 8 + 2 * t4) = pack_bf16(o[i][2 * r] * f, o[i][2 * r + 1] * f);
    }
}

// Single tokens (decoding): one CTA per (token, kv head, share of the key tiles).  The rows of the MMA tile are the
// query heads that share the kv head (up to 16); the four warps take a quarter of every tile's 64 keys each, with a
// running maximum and sum of their own, and are merged through shared memory at the end.  With several shares the
// merged (maximum, sum, weighted values) go to the workspace that attn_merge adds up.
constexpr int kDecStages = 3;       // key/value tiles in flight per CTA

template <int KD, int VD>
__global__ void __launch_bounds__(128)
gated_attn_mma_decode_kernel(const float* __restrict__ q, const bf16* __restrict__ k_pages, const bf16* __restrict__ v_pages,
                             const int* __restrict__ page_table, int table_stride, int ring_pages,
                             const float* __restrict__ sink, const float* __restrict__ gate, long long gate_stride,
                             const int* __restrict__ token_pos, const int* __restrict__ token_seq,
                             const int* __restrict__ seq_slot, void* __restrict__ out_v, int out_f32,
                             float* __restrict__ part_acc, float* __restrict__ part_ml, int n_splits, int H, int G,
                             float scale, int chunk, int window, int keep_first) {
    pdl_enter();
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* q_s = reinterpret_cast<bf16*>(smem_raw);                 // [16][KD]
    bf16* kv_s = q_s + 16 * KD;                                    // kDecStages stages: K [64][KD] then V [64][VD]
    constexpr int kStage = MK * (KD + VD);
    const int n = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
    const int QH = H / G, h0 = kvh * QH;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
    const int seq = token_seq[n];
    if (seq < 0) {                                                  // padding: defined rows, nothing read
        for (int idx = threadIdx.x; idx < QH * VD; idx += 128) {
            const size_t hrow = (size_t)n * H + h0 + idx / VD;
            if (n_splits == 1) {
                if (out_f32) ((float*)out_v)[hrow * VD + idx % VD] = 0.f;
                else ((bf16*)out_v)[hrow * VD + idx % VD] = from_float<bf16>(0.f);
            }
            else if (idx % VD == 0) {
                part_ml[(hrow * n_splits + split) * 2] = -INFINITY;
                part_ml[(hrow * n_splits + split) * 2 + 1] = 0.f;
            }
        }
        return;
    }
    const int pos = token_pos[n];
    int lo = chunk > 0 ? pos / chunk * chunk : 0;
    if (window > 0) lo = max(lo, pos + 1 - window);
    // the tiles a row sees, counted 0, 1, ...: the tiles of the kept first keys (those before the mask's own first
    // tile), then the mask's tiles; the shares are runs of that count
    const int kt_first = lo / MK;
    const int n_keep = keep_first > 0 ? min((keep_first + MK - 1) / MK, kt_first) : 0;
    const int n_all = n_keep + pos / MK - kt_first + 1;
    const int per = (n_all + n_splits - 1) / n_splits;
    const int kt_lo = split * per;
    const int n_kt = min(per, n_all - kt_lo);
    auto tile_of = [&](int i) { return i < n_keep ? i : kt_first + i - n_keep; };
    if (n_kt <= 0) {                                                // a share without tiles (never the first)
        for (int i = threadIdx.x; i < QH; i += 128) {
            const size_t pi = ((size_t)n * H + h0 + i) * n_splits + split;
            part_ml[pi * 2] = -INFINITY;
            part_ml[pi * 2 + 1] = 0.f;
        }
        return;
    }
    const int* table = page_table + (size_t)seq_slot[seq] * table_stride;
    for (int i = threadIdx.x; i < 16 * (KD / 8); i += 128) {
        const int r = i / (KD / 8), c = i % (KD / 8);
        uint4 packed = make_uint4(0u, 0u, 0u, 0u);
        if (r < QH) {
            const float* src = q + ((size_t)n * H + h0 + r) * KD + c * 8;
            const float4 a = *(const float4*)src, b = *(const float4*)(src + 4);
            packed = make_uint4(pack_bf16(a.x, a.y), pack_bf16(a.z, a.w), pack_bf16(b.x, b.y), pack_bf16(b.z, b.w));
        }
        *reinterpret_cast<uint4*>(q_s + tile_chunk_offset<KD>(r, c)) = packed;
    }
    auto load_kv = [&](int kt, int stage) {
        const int page = table[ring_pages > 0 ? kt % ring_pages : kt];
        const bf16* ksrc = k_pages + ((size_t)page * G + kvh) * (size_t)kPageTokens * KD;
        const bf16* vsrc = v_pages + ((size_t)page * G + kvh) * (size_t)kPageTokens * VD;
        bf16* ks = kv_s + (size_t)stage * kStage;
        bf16* vs = ks + MK * KD;
        for (int i = threadIdx.x; i < MK * (KD / 8); i += 128) cp16(ks + i * 8, ksrc + i * 8);
        for (int i = threadIdx.x; i < MK * (VD / 8); i += 128) cp16(vs + i * 8, vsrc + i * 8);
    };
    for (int s = 0; s < kDecStages - 1; ++s) {                      // the first tiles are on their way before anything else
        if (s < n_kt) load_kv(tile_of(kt_lo + s), s);
        cp_commit();
    }

    // the sink counts once: in the first share's first warp
    const bool with_sink = sink != nullptr && split == 0 && warp == 0;
    float m_run[2], l_run[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = g + 8 * r;
        m_run[r] = (with_sink && row < QH) ? sink[h0 + row] : -INFINITY;
        l_run[r] = (with_sink && row < QH && t4 == 0) ? 1.f : 0.f;
    }
    float o[VD / 8][4];
#pragma unroll
    for (int i = 0; i < VD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    const uint32_t q_base = smem_u32(q_s);

    for (int it = 0; it < n_kt; ++it) {
        const int stage = it % kDecStages;
        if (it + kDecStages - 1 < n_kt) load_kv(tile_of(kt_lo + it + kDecStages - 1), (it + kDecStages - 1) % kDecStages);
        cp_commit();
        cp_wait<kDecStages - 1>();
        __syncthreads();
        const uint32_t k_base = smem_u32(kv_s + (size_t)stage * kStage);
        const uint32_t v_base = k_base + 2 * MK * KD;
        const int key0 = tile_of(kt_lo + it) * MK + warp * 16;             // this warp's 16 keys of the tile

        float sc[2][4];
#pragma unroll
        for (int i = 0; i < 2; ++i) sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < KD / 16; ++kk) {
            uint32_t qa[4], b[4];
            ldmatrix_x4(qa, q_base + 2 * tile_chunk_offset<KD>((lane & 7) + ((lane >> 3) & 1) * 8, kk * 2 + (lane >> 4)));
            ldmatrix_x4(b, k_base + 2 * tile_chunk_offset<KD>(warp * 16 + (lane & 7) + (lane >> 4) * 8, kk * 2 + ((lane >> 3) & 1)));
            mma_bf16(sc[0], qa, b[0], b[1]);
            mma_bf16(sc[1], qa, b[2], b[3]);
        }
        float m_new[2] = {m_run[0], m_run[1]};
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int key = key0 + nt * 8 + 2 * t4 + (i & 1);
                const float s = (key <= pos && (key >= lo || key < keep_first)) ? sc[nt][i] * scale : -INFINITY;
                sc[nt][i] = s;
                m_new[i >> 1] = fmaxf(m_new[i >> 1], s);
            }
        float corr[2], m_use[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            m_new[r] = fmaxf(m_new[r], __shfl_xor_sync(0xffffffffu, m_new[r], 1));
            m_new[r] = fmaxf(m_new[r], __shfl_xor_sync(0xffffffffu, m_new[r], 2));
            m_use[r] = m_new[r] == -INFINITY ? 0.f : m_new[r];
            corr[r] = __expf(m_run[r] - m_use[r]);
            m_run[r] = m_new[r];
            l_run[r] *= corr[r];
        }
#pragma unroll
        for (int i = 0; i < VD / 8; ++i) {
            o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1];
        }
        uint32_t hi[4], lw[4];
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const float a = __expf(sc[h][2 * j] - m_use[j]), b = __expf(sc[h][2 * j + 1] - m_use[j]);
                l_run[j] += a + b;
                const float ah = __bfloat162float(__float2bfloat16_rn(a)), bh = __bfloat162float(__float2bfloat16_rn(b));
                hi[h * 2 + j] = pack_bf16(ah, bh);
                lw[h * 2 + j] = pack_bf16(a - ah, b - bh);
            }
#pragma unroll
        for (int dd = 0; dd < VD / 16; ++dd) {
            uint32_t vb[4];
            ldmatrix_x4_trans(vb, v_base + 2 * tile_chunk_offset<VD>(warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, dd * 2 + (lane >> 4)));
            mma_bf16(o[dd * 2], hi, vb[0], vb[1]);
            mma_bf16(o[dd * 2 + 1], hi, vb[2], vb[3]);
            mma_bf16(o[dd * 2], lw, vb[0], vb[1]);
            mma_bf16(o[dd * 2 + 1], lw, vb[2], vb[3]);
        }
        __syncthreads();
    }
    cp_wait<0>();
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    // the four warps' results side by side in shared memory (the stages are free), then merged per (head, column)
    float* mg = reinterpret_cast<float*>(kv_s);                     // [4][16][VD + 2]
    constexpr int kRow = VD + 2;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        float* dst = mg + ((size_t)warp * 16 + g + 8 * r) * kRow;
#pragma unroll
        for (int i = 0; i < VD / 8; ++i) {
            dst[i * 8 + 2 * t4] = o[i][2 * r];
            dst[i * 8 + 2 * t4 + 1] = o[i][2 * r + 1];
        }
        if (t4 == 0) {
            dst[VD] = m_run[r];
            dst[VD + 1] = l_run[r];
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < QH * VD; idx += 128) {
        const int row = idx / VD, d = idx % VD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) M = fmaxf(M, mg[((size_t)w * 16 + row) * kRow + VD]);
        float L = 0.f, A = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float* src = mg + ((size_t)w * 16 + row) * kRow;
            if (src[VD + 1] > 0.f) {
                const float e = __expf(src[VD] - M);
                L = fmaf(src[VD + 1], e, L);
                A = fmaf(src[d], e, A);
            }
        }
        const size_t hrow = (size_t)n * H + h0 + row;
        if (n_splits == 1) {
            float f = L > 0.f ? 1.f / L : 0.f;
            if (gate != nullptr) f *= 1.f / (1.f + expf(-gate[(size_t)n * gate_stride + h0 + row]));
            if (out_f32) ((float*)out_v)[hrow * VD + d] = A * f;
            else ((bf16*)out_v)[hrow * VD + d] = from_float<bf16>(A * f);
        } else {
            part_acc[(hrow * n_splits + split) * VD + d] = A;
            if (d == 0) {
                part_ml[(hrow * n_splits + split) * 2] = M;
                part_ml[(hrow * n_splits + split) * 2 + 1] = L;
            }
        }
    }
}

}  // namespace hos

using namespace hos;

// Head sizes of 64 or 128 numbers each (the caller runs the other kernel for the rest).
// q: float32 [N][H][kd]; out: [N][H][vd], bfloat16 or (out_f32) float32; n_q_tiles: at least the sum over sequences of
// ceil(rows / 64).
extern "C" int hos_gated_attn_mma(const float* q, const void* k_pages, const void* v_pages, const int* page_table,
                                  int table_stride, int ring_pages, const float* sink, const float* gate,
                                  long long gate_stride, const int* cu_seqlens, const int* token_pos, const int* token_seq,
                                  const int* seq_slot, void* out, int out_f32, int n_seqs, int n_q_tiles, int H, int G, int kd, int vd,
                                  float scale, int chunk, int window, int keep_first, cudaStream_t stream) {
    if (n_seqs <= 0 || n_q_tiles <= 0) return 0;
    if (G <= 0 || H % G != 0 || H > 65535) HOS_REFUSE("gated_attn_mma: %d heads over %d kv heads", H, G);
    if ((kd != 64 && kd != 128) || (vd != 64 && vd != 128))
        HOS_REFUSE("gated_attn_mma: heads of %d and %d numbers (64 or 128 are compiled)", kd, vd);
    if (((uintptr_t)q % 16) || ((uintptr_t)k_pages % 16) || ((uintptr_t)v_pages % 16) || ((uintptr_t)out % (out_f32 ? 8 : 4)))
        HOS_REFUSE("gated_attn_mma: rows and pages must be 16-byte aligned");
    const dim3 grid(n_q_tiles, H);
#define HOS_GAM(KDv, VDv)                                                                                            \
    do {                                                                                                             \
        constexpr int smem = (MQ * KDv + 2 * MK * (KDv + VDv)) * 2;                                                  \
        static bool attr_set = false;                                                                                \
        if (!attr_set) {                                                                                             \
            cudaFuncSetAttribute(gated_attn_mma_kernel<KDv, VDv>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); \
            attr_set = true;                                                                                         \
        }                                                                                                            \
        launch_pdl(gated_attn_mma_kernel<KDv, VDv>, grid, dim3(128), smem, stream, q, (const bf16*)k_pages,          \
                   (const bf16*)v_pages, page_table, table_stride, ring_pages, sink, gate, gate_stride, cu_seqlens,  \
                   token_pos, token_seq, seq_slot, out, out_f32, n_seqs, H, G, scale, chunk, window, keep_first);    \
    } while (0)
    if (kd == 64 && vd == 64) HOS_GAM(64, 64);
    else if (kd == 64) HOS_GAM(64, 128);
    else if (vd == 64) HOS_GAM(128, 64);
    else HOS_GAM(128, 128);
#undef HOS_GAM
    return check_launch("gated_attn_mma");
}

// Single tokens: q float32 [N][H][kd], out [N][H][vd] bfloat16 or (out_f32) float32; up to 16 query heads to a kv head.  With n_splits > 1 the
// shares' partial results go to part_acc [N][H][n_splits][vd] and part_ml [N][H][n_splits][2] for hos_attn_merge.
extern "C" int hos_gated_attn_mma_decode(const float* q, const void* k_pages, const void* v_pages, const int* page_table,
                                         int table_stride, int ring_pages, const float* sink, const float* gate,
                                         long long gate_stride, const int* token_pos, const int* token_seq,
                                         const int* seq_slot, void* out, int out_f32, float* part_acc, float* part_ml,
                                         int n_splits, int N, int H, int G, int kd, int vd, float scale, int chunk, int window,
                                         int keep_first, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (G <= 0 || H % G != 0 || H / G > 16 || G > 65535) HOS_REFUSE("gated_attn_mma_decode: %d heads over %d kv heads", H, G);
    if ((kd != 64 && kd != 128) || (vd != 64 && vd != 128))
        HOS_REFUSE("gated_attn_mma_decode: heads of %d and %d numbers (64 or 128 are compiled)", kd, vd);
    if (n_splits < 1 || n_splits > 65535 || (n_splits > 1 && (part_acc == nullptr || part_ml == nullptr)))
        HOS_REFUSE("gated_attn_mma_decode: %d shares need a workspace", n_splits);
    const dim3 grid(N, G, n_splits);
#define HOS_GAD(KDv, VDv)                                                                                            \
    do {                                                                                                             \
        constexpr int smem = (16 * KDv + kDecStages * MK * (KDv + VDv)) * 2;                                         \
        static_assert(4 * 16 * (VDv + 2) * 4 <= kDecStages * MK * (KDv + VDv) * 2, "the merge fits the stages");    \
        static bool attr_set = false;                                                                                \
        if (!attr_set) {                                                                                             \
            cudaFuncSetAttribute(gated_attn_mma_decode_kernel<KDv, VDv>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); \
            attr_set = true;                                                                                         \
        }                                                                                                            \
        launch_pdl(gated_attn_mma_decode_kernel<KDv, VDv>, grid, dim3(128), smem, stream, q, (const bf16*)k_pages,   \
                   (const bf16*)v_pages, page_table, table_stride, ring_pages, sink, gate, gate_stride, token_pos,   \
                   token_seq, seq_slot, out, out_f32, part_acc, part_ml, n_splits, H, G, scale, chunk, window,       \
                   keep_first);                                                                                      \
    } while (0)
    if (kd == 64 && vd == 64) HOS_GAD(64, 64);
    else if (kd == 64) HOS_GAD(64, 128);
    else if (vd == 64) HOS_GAD(128, 64);
    else HOS_GAD(128, 128);
#undef HOS_GAD
    return check_launch("gated_attn_mma_decode");
}
