// Linear recurrences with a matrix state per head, S [dim keys][vdim values] in 32-bit, one kernel for two rules:
//
//   decay rule   S <- g S + k v^T                                o = S^T q     (g a constant per head)
//   delta rule   S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q  (g, beta per token and head)
//
// The read-out sees the current token's write.  A sequence's state lives per slot as S^T ([head][vdim][dim]: a
// thread's run of rows of one column is contiguous), starts at zero (a sequence whose first row is position 0
// ignores what the slot holds), and is carried from step to step.
//
// state_scan: one block per (sequence, head, run of value columns); a column of S is cut into R runs of DR rows,
//   one thread each (R lanes side by side, so that sums over a column are shuffles); tokens in order, a chunk of
//   them staged in shared memory while the chunk before it is walked (cp.async, two buffers).  Columns are
//   independent of one another in both rules.
// act_rows: x logistic(x) in place on the leading columns of 32-bit rows (the decay rule's q, k, v).
// rotate_rows: rotary positions in place on the q and k heads of 32-bit rows (either pairing, the first rot_dims
//   numbers of a head; angle = position * freq in 32-bit, sincosf), the keys then multiplied by a constant.
// conv_prep (the delta rule's inputs): per token, the short causal convolution over time of the q, k, v
//   projections (per channel, `taps` wide, the last tap the current token's, the inputs before a step's first
//   row from the slot's state), x sigmoid(x) of it, q and k divided by their length per head
//   (sqrt(sum + 1e-6)), q times dim^-1/2; beta = logistic(b); g = exp(-exp(A_log) softplus(a + dt_bias)).
// conv_keep: the last taps - 1 inputs of every sequence go to the slot's state.
#include "common.cuh"

namespace hos {

constexpr int kScanChunk = 8;       // tokens staged at a time
constexpr int kPad = 4;             // floats after every DR staged numbers: 16-byte reads of R neighbours miss each other's banks

__device__ __forceinline__ float silu_precise(float x) { return x / (1.f + expf(-x)); }

__device__ __forceinline__ void cp_async4(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit_all() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// x <- x logistic(x) on the first `cols` numbers of every row (the decay rule's q, k, v before the scan)
__global__ void act_rows_kernel(float* __restrict__ x, long long ld, int cols, long long n) {
    pdl_enter();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float* p = x + (i / cols) * ld + (i % cols);
    *p = silu_precise(*p);
}

// x: float32 [N][ld]; from column 0 on `Hq` query heads and then `Hk` key heads of `dim` numbers each.  The first
// rot_dims numbers of every head turn with the token's position: style 0 pairs number i with i + rot_dims / 2,
// style 1 number 2i with 2i + 1; (u, v) -> (u cos a - v sin a, v cos a + u sin a), a = position * freq[i].  Every
// number of a key head is then multiplied by k_mult.  An item is one pair, or one number beyond rot_dims.
__global__ void __launch_bounds__(256)
rotate_rows_kernel(float* __restrict__ x, long long ld, int Hq, int Hk, int dim, int rot_dims, int style,
                   const float* __restrict__ freq, const int* __restrict__ token_pos, const int* __restrict__ token_seq,
                   float k_mult) {
    pdl_enter();
    extern __shared__ float2 rot_tab[];          // [rot_dims / 2] (sine, cosine) of this token
    const int n = blockIdx.x;
    if (token_seq[n] < 0) return;
    const float fpos = (float)token_pos[n];
    const int half = rot_dims >> 1;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float sn, cs;
        sincosf(fpos * freq[i], &sn, &cs);
        rot_tab[i] = make_float2(sn, cs);
    }
    __syncthreads();
    float* row = x + (size_t)n * ld;
    const int per = half + (dim - rot_dims);
    for (int it = threadIdx.x; it < (Hq + Hk) * per; it += blockDim.x) {
        const int head = it / per, j = it - head * per;
        const float m = head >= Hq ? k_mult : 1.f;
        float* hp = row + (size_t)head * dim;
        if (j < half) {
            const int a = style == 0 ? j : 2 * j, b = style == 0 ? j + half : 2 * j + 1;
            const float2 sc = rot_tab[j];
            const float u = hp[a], v = hp[b];
            hp[a] = (u * sc.y - v * sc.x) * m;
            hp[b] = (v * sc.y + u * sc.x) * m;
        } else if (m != 1.f) {
            hp[rot_dims + (j - half)] *= m;
        }
    }
}

template <int DR, int R, bool DELTA>
__global__ void __launch_bounds__(256)
state_scan_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v, long long ld,
                  int aligned, int act_in_walk, const float* __restrict__ g, long long g_ld, const float* __restrict__ beta,
                  long long beta_ld, float* __restrict__ state, const int* __restrict__ token_pos,
                  const int* __restrict__ token_seq, const int* __restrict__ cu_seqlens, const int* __restrict__ seq_slot,
                  float* __restrict__ out, int H, int Gk, int dim, int vdim, int CC, const float* __restrict__ rot_freq,
                  int rot_dims, int rot_style, float k_mult) {
    pdl_enter();
    extern __shared__ __align__(16) float sm[];
    const int seq = blockIdx.x, head = blockIdx.y, col0 = blockIdx.z * CC;
    const int lo = cu_seqlens[seq], hi = cu_seqlens[seq + 1];
    if (hi <= lo || token_seq[lo] < 0) return;
    const int slot = seq_slot[seq];
    const int kh = head / (H / Gk);
    const int r = threadIdx.x % R, c = threadIdx.x / R;
    const int col = col0 + c;
    const bool rot_in_walk = rot_dims > 0 || k_mult != 1.f;
    const bool live = c < CC && col < vdim;
    const int dpad = R * (DR + kPad);
    // two buffers of staged tokens: while one chunk is walked the next one's rows are on their way (cp.async)
    const int per_buf = kScanChunk * (2 * dpad + 2 * CC) + 2 * kScanChunk;      // q, k, v, o, g, beta
    const int CC4 = (CC + 3) & ~3;
    (void)CC4;

    float S[DR];
    float* st = state + (((size_t)slot * H + head) * vdim + (live ? col : 0)) * dim + r * DR;
    const bool fresh = token_pos[lo] == 0;
    // a thread's run of rows is contiguous in the kept S^T: 16 bytes at a time where the run is whole and aligned
    const bool whole = live && r * DR + DR <= dim && (dim & 3) == 0;
    if (!fresh && whole) {
#pragma unroll
        for (int i = 0; i < DR / 4; ++i) {
            const float4 t = ((const float4*)st)[i];
            S[4 * i] = t.x; S[4 * i + 1] = t.y; S[4 * i + 2] = t.z; S[4 * i + 3] = t.w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < DR; ++i) S[i] = (!fresh && live && r * DR + i < dim) ? st[i] : 0.f;
    }
    // rows beyond dim and columns beyond vdim are read by the walk and never staged: they stay zero for good
    if (R * DR != dim || col0 + CC > vdim) {
        for (int i = threadIdx.x; i < 2 * per_buf; i += blockDim.x) sm[i] = 0.f;
        __syncthreads();
    }

    auto stage = [&](int t0, int nt, float* buf) {
        float* qs = buf;
        float* ks = qs + kScanChunk * dpad;
        float* vs = ks + kScanChunk * dpad;
        float* gs = vs + 2 * kScanChunk * CC;        // after v and o
        float* bs = gs + kScanChunk;
        if (aligned) {
            const int d4 = dim >> 2;
            for (int idx = threadIdx.x; idx < nt * d4; idx += blockDim.x) {
                const int t = idx / d4, d = (idx % d4) << 2;
                const int at = t * dpad + d + (d / DR) * kPad;
                cp_async16(qs + at, q + (size_t)(t0 + t) * ld + kh * dim + d);
                cp_async16(ks + at, k + (size_t)(t0 + t) * ld + kh * dim + d);
            }
        } else {
            for (int idx = threadIdx.x; idx < nt * dim; idx += blockDim.x) {
                const int t = idx / dim, d = idx % dim;
                const int at = t * dpad + d + (d / DR) * kPad;
                cp_async4(qs + at, q + (size_t)(t0 + t) * ld + kh * dim + d);
                cp_async4(ks + at, k + (size_t)(t0 + t) * ld + kh * dim + d);
            }
        }
        const int ncol = min(CC, vdim - col0);
        for (int idx = threadIdx.x; idx < nt * ncol; idx += blockDim.x) {
            const int t = idx / ncol, cc = idx % ncol;
            cp_async4(vs + t * CC + cc, v + (size_t)(t0 + t) * ld + head * vdim + col0 + cc);
        }
        if (threadIdx.x < nt) {
            cp_async4(gs + threadIdx.x, g + (size_t)(t0 + threadIdx.x) * g_ld + head);
            if (DELTA) cp_async4(bs + threadIdx.x, beta + (size_t)(t0 + threadIdx.x) * beta_ld + head);
        }
        cp_async_commit_all();
    };

    stage(lo, min(kScanChunk, hi - lo), sm);
    int which = 0;
    for (int t0 = lo; t0 < hi; t0 += kScanChunk, which ^= 1) {
        const int nt = min(kScanChunk, hi - t0);
        cp_async_wait_all();
        __syncthreads();            // this chunk has landed; everyone is done with the other buffer
        if (t0 + kScanChunk < hi) stage(t0 + kScanChunk, min(kScanChunk, hi - t0 - kScanChunk), sm + (which ^ 1) * per_buf);
        float* qs = sm + which * per_buf;
        float* ks = qs + kScanChunk * dpad;
        if (rot_in_walk) {
            // the staged q and k turn with their tokens' positions, and the keys take their factor, as rotate_rows would
            // have done in a launch of its own (meant for single-token steps: every block of a head repeats it)
            const int half = rot_dims >> 1, per = half + (dim - rot_dims);
            for (int idx = threadIdx.x; idx < nt * per; idx += blockDim.x) {
                const int t = idx / per, j = idx - t * per;
                float* qp = qs + t * dpad;
                float* kp = ks + t * dpad;
                if (j < half) {
                    const int a = rot_style == 0 ? j : 2 * j, b = rot_style == 0 ? j + half : 2 * j + 1;
                    const int ia = a + (a / DR) * kPad, ib = b + (b / DR) * kPad;
                    float sn, cs;
                    sincosf((float)token_pos[t0 + t] * rot_freq[j], &sn, &cs);
                    const float qu = qp[ia], qv = qp[ib], ku = kp[ia], kv = kp[ib];
                    qp[ia] = qu * cs - qv * sn;
                    qp[ib] = qv * cs + qu * sn;
                    kp[ia] = (ku * cs - kv * sn) * k_mult;
                    kp[ib] = (kv * cs + ku * sn) * k_mult;
                } else {
                    const int d = rot_dims + (j - half);
                    kp[d + (d / DR) * kPad] *= k_mult;
                }
            }
            __syncthreads();
        }
        float* vs = ks + kScanChunk * dpad;
        float* os = vs + kScanChunk * CC;
        float* gs = os + kScanChunk * CC;
        float* bs = gs + kScanChunk;
        {       // every thread walks (a warp's shuffles want all its lanes); only live columns are written
            float part[kScanChunk];       // the read-outs' partial sums: added up after the walk, off its chain
#pragma unroll
            for (int t = 0; t < kScanChunk; ++t) {
                part[t] = 0.f;
                if (t >= nt) continue;
                const float4* k4 = (const float4*)(ks + t * dpad + r * (DR + kPad));
                const float4* q4 = (const float4*)(qs + t * dpad + r * (DR + kPad));
                const float gt = gs[t];
                float u = c < CC ? vs[t * CC + c] : 0.f;
                if (!DELTA && act_in_walk) u = silu_precise(u);      // single tokens: the activation rides here
                if (DELTA) {
                    float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;       // four chains, not one of DR links
#pragma unroll
                    for (int i = 0; i < DR / 4; ++i) {
                        const float4 kk = k4[i];
                        S[4 * i] *= gt; S[4 * i + 1] *= gt; S[4 * i + 2] *= gt; S[4 * i + 3] *= gt;
                        d0 = fmaf(S[4 * i], kk.x, d0);
                        d1 = fmaf(S[4 * i + 1], kk.y, d1);
                        d2 = fmaf(S[4 * i + 2], kk.z, d2);
                        d3 = fmaf(S[4 * i + 3], kk.w, d3);
                    }
                    float dot = (d0 + d1) + (d2 + d3);
#pragma unroll
                    for (int o = 1; o < R; o <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
                    u = bs[t] * (u - dot);
                }
                float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
                for (int i = 0; i < DR / 4; ++i) {
                    float4 kk = k4[i], qq = q4[i];
                    if (!DELTA && act_in_walk) {
                        kk = make_float4(silu_precise(kk.x), silu_precise(kk.y), silu_precise(kk.z), silu_precise(kk.w));
                        qq = make_float4(silu_precise(qq.x), silu_precise(qq.y), silu_precise(qq.z), silu_precise(qq.w));
                    }
                    if (DELTA) {
                        S[4 * i] = fmaf(kk.x, u, S[4 * i]);
                        S[4 * i + 1] = fmaf(kk.y, u, S[4 * i + 1]);
                        S[4 * i + 2] = fmaf(kk.z, u, S[4 * i + 2]);
                        S[4 * i + 3] = fmaf(kk.w, u, S[4 * i + 3]);
                    } else {
                        S[4 * i] = fmaf(gt, S[4 * i], kk.x * u);
                        S[4 * i + 1] = fmaf(gt, S[4 * i + 1], kk.y * u);
                        S[4 * i + 2] = fmaf(gt, S[4 * i + 2], kk.z * u);
                        S[4 * i + 3] = fmaf(gt, S[4 * i + 3], kk.w * u);
                    }
                    a0 = fmaf(S[4 * i], qq.x, a0);
                    a1 = fmaf(S[4 * i + 1], qq.y, a1);
                    a2 = fmaf(S[4 * i + 2], qq.z, a2);
                    a3 = fmaf(S[4 * i + 3], qq.w, a3);
                }
                part[t] = (a0 + a1) + (a2 + a3);
            }
#pragma unroll
            for (int t = 0; t < kScanChunk; ++t) {
                if (t >= nt) break;
                float acc = part[t];
#pragma unroll
                for (int o = 1; o < R; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
                if (r == 0 && c < CC) os[t * CC + c] = acc;
            }
        }
        __syncthreads();
        for (int idx = threadIdx.x; idx < nt * CC; idx += blockDim.x) {
            const int t = idx / CC, cc = idx % CC;
            if (col0 + cc < vdim) out[((size_t)(t0 + t) * H + head) * vdim + col0 + cc] = os[idx];
        }
    }
    if (whole) {
#pragma unroll
        for (int i = 0; i < DR / 4; ++i) ((float4*)st)[i] = make_float4(S[4 * i], S[4 * i + 1], S[4 * i + 2], S[4 * i + 3]);
    } else if (live) {
#pragma unroll
        for (int i = 0; i < DR; ++i)
            if (r * DR + i < dim) st[i] = S[i];
    }
}

constexpr int kMaxTaps = 16;

// raw: float32 [N][ld]: q (Gk * dim) | k (Gk * dim) | v (H * vdim) | b (H) | a (H) | ... ; conv_w: [C][taps] over
// the first C = 2 Gk dim + H vdim columns; conv_state: [slots][taps - 1][C], row j the input taps - 1 - j tokens back.
__global__ void __launch_bounds__(256)
conv_prep_kernel(const float* __restrict__ raw, long long ld, const float* __restrict__ conv_w, int taps,
                 const float* conv_state,      // may be written through keep_here: neither is __restrict__
                 const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                 const int* __restrict__ token_pos, const int* __restrict__ token_seq, const int* __restrict__ cu_seqlens,
                 const int* __restrict__ seq_slot, float* __restrict__ act, float* __restrict__ beta_out,
                 float* __restrict__ g_out, int H, int Gk, int dim, int vdim, float* keep_here) {
    pdl_enter();
    extern __shared__ float qk[];                // [2 Gk dim] after the activation
    __shared__ float inv_len[64];
    const int n = blockIdx.x;
    const int seq = token_seq[n];
    const int QK = 2 * Gk * dim, C = QK + H * vdim;
    float* arow = act + (size_t)n * C;
    if (seq < 0) {
        for (int i = threadIdx.x; i < C; i += blockDim.x) arow[i] = 0.f;
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            beta_out[(size_t)n * H + i] = 0.f;
            g_out[(size_t)n * H + i] = 1.f;
        }
        return;
    }
    const int r0 = cu_seqlens[seq];
    const bool fresh = token_pos[r0] == 0;
    const float* keep = conv_state + (size_t)seq_slot[seq] * (taps - 1) * C;
    // keep_here: every sequence of the step brings one token, so this block alone reads and writes its slot's kept
    // inputs (a thread the channels it convolves): they move on by one here instead of in a launch of their own
    float* keep_w = keep_here != nullptr ? keep_here + (size_t)seq_slot[seq] * (taps - 1) * C : nullptr;
    for (int ch = threadIdx.x; ch < C; ch += blockDim.x) {
        float acc = 0.f;
        for (int j = 0; j < taps; ++j) {
            const int src = n - (taps - 1) + j;          // the row of this step that holds the input, if it is one
            float x = 0.f;
            if (src >= r0) x = raw[(size_t)src * ld + ch];
            else if (!fresh) x = keep[(size_t)((taps - 1) + (src - r0)) * C + ch];
            acc = fmaf(conv_w[(size_t)ch * taps + j], x, acc);
            if (keep_w != nullptr && j >= 1) keep_w[(size_t)(j - 1) * C + ch] = x;      // row j - 1 is read before this
        }
        const float y = silu_precise(acc);
        if (ch < QK) qk[ch] = y;
        else arow[ch] = y;
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    for (int hd0 = 0; hd0 < 2 * Gk; hd0 += 64) {         // the heads' lengths, a warp per head
        for (int hd = hd0 + warp; hd < min(2 * Gk, hd0 + 64); hd += nwarps) {
            float ss = 0.f;
            for (int d = lane; d < dim; d += 32) ss = fmaf(qk[hd * dim + d], qk[hd * dim + d], ss);
            ss = warp_sum(ss);
            if (lane == 0) inv_len[hd - hd0] = (1.f / sqrtf(ss + 1e-6f)) * (hd < Gk ? 1.f / sqrtf((float)dim) : 1.f);
        }
        __syncthreads();
        for (int i = hd0 * dim + threadIdx.x; i < min(2 * Gk, hd0 + 64) * dim; i += blockDim.x)
            arow[i] = qk[i] * inv_len[i / dim - hd0];
        __syncthreads();
    }
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
        const float b = raw[(size_t)n * ld + C + h], a = raw[(size_t)n * ld + C + H + h] + dt_bias[h];
        beta_out[(size_t)n * H + h] = 1.f / (1.f + expf(-b));
        const float sp = a > 20.f ? a : log1pf(expf(a));
        g_out[(size_t)n * H + h] = expf(-expf(a_log[h]) * sp);
    }
}

__global__ void conv_keep_kernel(const float* __restrict__ raw, long long ld, int taps, float* __restrict__ conv_state,
                                 const int* __restrict__ token_pos, const int* __restrict__ token_seq,
                                 const int* __restrict__ cu_seqlens, const int* __restrict__ seq_slot, int C) {
    pdl_enter();
    const int seq = blockIdx.y;
    const int ch = blockIdx.x * blockDim.x + threadIdx.x;
    const int r0 = cu_seqlens[seq], r1 = cu_seqlens[seq + 1];
    if (ch >= C || r1 <= r0 || token_seq[r0] < 0) return;
    const bool fresh = token_pos[r0] == 0;
    float* keep = conv_state + (size_t)seq_slot[seq] * (taps - 1) * C;
    float nv[kMaxTaps];
#pragma unroll
    for (int j = 0; j < kMaxTaps; ++j) {
        if (j < taps - 1) {
            const int src = r1 - (taps - 1) + j;
            nv[j] = src >= r0 ? raw[(size_t)src * ld + ch] : (fresh ? 0.f : keep[(size_t)((taps - 1) + (src - r0)) * C + ch]);
        }
    }
#pragma unroll
    for (int j = 0; j < kMaxTaps; ++j)
        if (j < taps - 1) keep[(size_t)j * C + ch] = nv[j];
}

}  // namespace hos

using namespace hos;

// q, k: rows of Gk heads of `dim` numbers; v: rows of H heads of `vdim`; all float32 with `ld` numbers between rows.
// g: [.][H] with g_ld between rows (0: one row of constants).  beta: null for the decay rule.  state: [slots][H][vdim][dim].
// out: float32 [N][H][vdim].  act_in_walk (decay rule only, meant for single-token steps): q, k, v are taken through
// x logistic(x) as they are read, instead of by hos_act_rows before.  rot_freq ([rot_dims / 2], or null), rot_style, k_mult:
// the staged q and k are turned by their tokens' positions and the keys multiplied, as hos_rotate_rows would have done
// before (meant for single-token steps; it follows the rows as they are, so it does not go with act_in_walk).
extern "C" int hos_state_scan(const float* q, const float* k, const float* v, long long ld, int act_in_walk, const float* g,
                              long long g_ld, const float* beta, long long beta_ld, float* state, const int* token_pos,
                              const int* token_seq, const int* cu_seqlens, const int* seq_slot, float* out, int n_rows,
                              int n_seqs, int H, int Gk, int dim, int vdim, const float* rot_freq, int rot_dims, int rot_style,
                              float k_mult, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (rot_freq == nullptr) rot_dims = 0;
    if (rot_dims < 0 || rot_dims % 2 != 0 || rot_dims > dim || (rot_style != 0 && rot_style != 1))
        HOS_REFUSE("state_scan: %d rotated numbers in heads of %d", rot_dims, dim);
    if (Gk <= 0 || H % Gk != 0) HOS_REFUSE("state_scan: %d heads are not a multiple of %d key heads", H, Gk);
    if (dim <= 0 || dim > 1024 || vdim <= 0) HOS_REFUSE("state_scan: heads of %d x %d", dim, vdim);
    // short runs of rows per thread: a token's walk is a chain of dependent instructions (scale, dot, sum over the
    // runs, update, read-out, sum), and with few (sequence, head) pairs nothing else hides its latency; the sums over
    // 16 or 32 runs are shuffles
    // (heads of 128 x 128, 2,048 tokens, decay / delta rule: 4 rows to a thread 477 / 628 us, 8 rows 459 / 598, 16 rows
    // 584 / 679, 32 rows 900 / 961)
    const int DR = dim <= 16 ? 4 : (dim <= 256 ? 8 : (dim <= 512 ? 16 : 32));
    int R = 1;
    while (R * DR < dim) R <<= 1;
    if (DR == 8 && R < 4) R = 4;          // the compiled shapes (rows beyond dim are zeros)
    if (DR >= 16) R = 32;
    int CC = 256 / R;
    if (CC > vdim) CC = vdim;
    // single tokens and few (sequence, head) pairs: fewer columns to a block, so that the blocks fill the GPU (columns
    // are independent; every block stages the whole q and k rows, which a long walk would pay for token by token)
    if (n_rows <= 2 * n_seqs)
        while (CC * R > 64 && (long long)n_seqs * H * ((vdim + CC - 1) / CC) < 2 * sm_count_cached()) CC = (CC + 1) / 2;
    const int threads = (CC * R + 31) / 32 * 32;
    const int dpad = R * (DR + kPad);
    const size_t smem = (size_t)2 * (2 * kScanChunk * dpad + 2 * kScanChunk * CC + 2 * kScanChunk) * sizeof(float);
    const int aligned = (dim % 4 == 0 && ld % 4 == 0 && (uintptr_t)q % 16 == 0 && (uintptr_t)k % 16 == 0) ? 1 : 0;
    const dim3 grid(n_seqs, H, (vdim + CC - 1) / CC);
    const bool delta = beta != nullptr;
    if (delta && act_in_walk) HOS_REFUSE("state_scan: the activation in the walk is the decay rule's");
    if (smem > 200 * 1024) HOS_REFUSE("state_scan: heads of %d x %d do not fit a block's shared memory", dim, vdim);
#define HOS_SCAN(DRv, Rv, DL)                                                                                        \
    do {                                                                                                             \
        if (smem > 48 * 1024)                                                                                        \
            cudaFuncSetAttribute(state_scan_kernel<DRv, Rv, DL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        launch_pdl(state_scan_kernel<DRv, Rv, DL>, grid, dim3(threads), smem, stream, q, k, v, ld, aligned, act_in_walk, g, g_ld, beta, \
                   beta_ld, state, token_pos, token_seq, cu_seqlens, seq_slot, out, H, Gk, dim, vdim, CC, rot_freq,  \
                   rot_dims, rot_style, k_mult);                                                                     \
    } while (0)
#define HOS_SCAN_D(DRv, Rv)                                                                                          \
    do {                                                                                                             \
        if (delta) HOS_SCAN(DRv, Rv, true);                                                                          \
        else HOS_SCAN(DRv, Rv, false);                                                                               \
    } while (0)
    // the shapes that the choice of DR above can give: (4; 1, 2, 4), (8; 4 to 32), (16; 32), (32; 32)
    if (DR == 4 && R == 1) HOS_SCAN_D(4, 1);
    else if (DR == 4 && R == 2) HOS_SCAN_D(4, 2);
    else if (DR == 4) HOS_SCAN_D(4, 4);
    else if (DR == 8 && R <= 4) HOS_SCAN_D(8, 4);
    else if (DR == 8 && R == 8) HOS_SCAN_D(8, 8);
    else if (DR == 8 && R == 16) HOS_SCAN_D(8, 16);
    else if (DR == 8) HOS_SCAN_D(8, 32);
    else if (DR == 16) HOS_SCAN_D(16, 32);
    else HOS_SCAN_D(32, 32);
#undef HOS_SCAN_D
#undef HOS_SCAN
    return check_launch("state_scan");
}

extern "C" int hos_act_rows(float* x, long long ld, int cols, int N, cudaStream_t stream) {
    const long long n = (long long)N * cols;
    if (n <= 0) return 0;
    launch_pdl(act_rows_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, x, ld, cols, n);
    return check_launch("act_rows");
}

// x: float32 rows of ld numbers whose first (Hq + Hk) * dim columns are the query heads and then the key heads; freq:
// [rot_dims / 2] or null (no rotation: only the keys' multiplier is applied); style 0: halves, 1: neighbours.
extern "C" int hos_rotate_rows(float* x, long long ld, int Hq, int Hk, int dim, int rot_dims, int style, const float* freq,
                               const int* token_pos, const int* token_seq, float k_mult, int N, cudaStream_t stream) {
    if (N <= 0 || Hq + Hk <= 0) return 0;
    if (freq == nullptr) rot_dims = 0;
    if (rot_dims < 0 || rot_dims % 2 != 0 || rot_dims > dim) HOS_REFUSE("rotate_rows: %d rotated numbers in heads of %d", rot_dims, dim);
    if (style != 0 && style != 1) HOS_REFUSE("rotate_rows: unknown pairing %d", style);
    if (rot_dims == 0 && k_mult == 1.f) return 0;
    const size_t smem = (size_t)(rot_dims / 2 + 1) * sizeof(float2);
    if (smem > 48 * 1024) HOS_REFUSE("rotate_rows: %d rotated numbers do not fit", rot_dims);
    launch_pdl(rotate_rows_kernel, dim3(N), dim3(256), smem, stream, x, ld, Hq, Hk, dim, rot_dims, style, freq, token_pos,
               token_seq, k_mult);
    return check_launch("rotate_rows");
}

// keep_here: 1 only where every sequence of the step brings exactly one token: the kept inputs then move on inside this
// launch and hos_conv_keep is not needed.
// act: float32 [N][2 Gk dim + H vdim] (q, k, v after convolution, activation and lengths); beta_out, g_out: [N][H].
extern "C" int hos_conv_prep(const float* raw, long long ld, const float* conv_w, int taps, const float* conv_state,
                             const float* a_log, const float* dt_bias, const int* token_pos, const int* token_seq,
                             const int* cu_seqlens, const int* seq_slot, float* act, float* beta_out, float* g_out, int N,
                             int H, int Gk, int dim, int vdim, int keep_here, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (taps < 1 || taps > kMaxTaps) HOS_REFUSE("conv_prep: %d taps are outside 1..%d", taps, kMaxTaps);
    const size_t smem = (size_t)2 * Gk * dim * sizeof(float);
    if (smem > 160 * 1024) HOS_REFUSE("conv_prep: %d query and key channels do not fit", 2 * Gk * dim);
    if (smem > 48 * 1024) cudaFuncSetAttribute(conv_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_pdl(conv_prep_kernel, dim3(N), dim3(256), smem, stream, raw, ld, conv_w, taps, conv_state, a_log, dt_bias,
               token_pos, token_seq, cu_seqlens, seq_slot, act, beta_out, g_out, H, Gk, dim, vdim,
               keep_here ? const_cast<float*>(conv_state) : (float*)nullptr);
    return check_launch("conv_prep");
}

extern "C" int hos_conv_keep(const float* raw, long long ld, int taps, float* conv_state, const int* token_pos,
                             const int* token_seq, const int* cu_seqlens, const int* seq_slot, int n_seqs, int C,
                             cudaStream_t stream) {
    if (n_seqs <= 0 || taps <= 1) return 0;
    if (taps > kMaxTaps) HOS_REFUSE("conv_keep: %d taps are outside 1..%d", taps, kMaxTaps);
    launch_pdl(conv_keep_kernel, dim3((C + 127) / 128, n_seqs), dim3(128), 0, stream, raw, ld, taps, conv_state, token_pos,
               token_seq, cu_seqlens, seq_slot, C);
    return check_launch("conv_keep");
}
