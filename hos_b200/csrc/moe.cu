// A routed feed-forward (mixture of experts) whose whole step stays on the device.
//
//   route     per row: router logits in 32-bit, scores = softmax over all outputs (or, scoring 1, the logistic
//             function of each logit), the `top` largest of (score + correction) chosen, each weighted by
//             its plain score (not renormalised).
//             The last `n_identity` router outputs are experts without tensors: their output is
//             the row itself.
//   align     the chosen (row, choice) pairs listed expert by expert, each expert's list padded to
//             whole tiles of kTile rows, and the expert of every tile.
//   gate_up   per tile, the expert's gate and up products of the listed rows and the activation
//             y = g' * sigmoid(alpha * g') * (u' + 1), g' = min(g, limit), u' = clamp(u, -limit, limit)
//             (limit <= 0: no clamp; the 1 is `up_shift`, 0 for the plain gated form g' sigmoid(alpha g') u').  With
//             in_weight the pair's weight multiplies the expert's INPUT: gate and up products are linear, so
//             g and u are multiplied by it before the activation, and down takes no weight.
//   down      per tile, the expert's down product, times the pair's weight, to the pair's own row
//             of a 32-bit buffer.
//   combine   per row, the sum of its pairs' rows in the order of the choices, identity experts added
//             as weight * row, plus the row of `extra` if given (an expert that every row uses).
// The grid of the tiled kernels is the most tiles the step can have; tiles beyond the real ones
// leave at once, so nothing depends on the host knowing the counts.  Products accumulate in 32-bit;
// a warp whose rows of a tile are all padding skips the arithmetic.
#include "common.cuh"
#include "mma_tile.cuh"

namespace hos {

__device__ __forceinline__ float4 route_load4(const float* p) { return *(const float4*)p; }
__device__ __forceinline__ float4 route_load4(const bf16* p) {
    const uint2 u = *(const uint2*)p;
    return make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xffff0000u), __uint_as_float(u.y << 16),
                       __uint_as_float(u.y & 0xffff0000u));
}

// One warp: z [n_out] logits of row n (in shared memory) -> scores, the `top` largest of (score + correction)
// and their plain scores.  A padding row (token_seq < 0) chooses nothing.
__device__ __forceinline__ void route_choose(float* z, float* taken, const float* __restrict__ correction,
                                             const int* __restrict__ token_seq, int* __restrict__ choice,
                                             float* __restrict__ weight, int n, int n_out, int top, int scoring, int lane,
                                             float renorm, float wscale) {
    if (token_seq[n] < 0) {
        for (int k = lane; k < top; k += 32) {
            choice[(size_t)n * top + k] = -1;
            weight[(size_t)n * top + k] = 0.f;
        }
        return;
    }
    // Logistic scores without a correction are ranked by their logits: the order is the scores' own, and it still tells
    // apart logits whose scores round to the same 32-bit number near 1.
    const bool by_logit = scoring == 1 && correction == nullptr;
    if (by_logit) {
    } else if (scoring == 1) {
        for (int e = lane; e < n_out; e += 32) z[e] = 1.f / (1.f + expf(-z[e]));
    } else {
        float m = -INFINITY;
        for (int e = lane; e < n_out; e += 32) m = fmaxf(m, z[e]);
        m = warp_max(m);
        float sum = 0.f;
        for (int e = lane; e < n_out; e += 32) {
            const float p = expf(z[e] - m);
            z[e] = p;
            sum += p;
        }
        sum = warp_sum(sum);
        __syncwarp();
        for (int e = lane; e < n_out; e += 32) z[e] = z[e] / sum;
    }
    __syncwarp();
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int arg = 0x7fffffff;
        for (int e = lane; e < n_out; e += 32) {
            if (taken[e] != 0.f) continue;
            const float c = z[e] + (correction ? correction[e] : 0.f);
            if (c > best || (c == best && e < arg)) {
                best = c;
                arg = e;
            }
        }
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ob > best || (ob == best && oa < arg)) {
                best = ob;
                arg = oa;
            }
        }
        if (lane == 0) {
            const bool ok = arg != 0x7fffffff;
            choice[(size_t)n * top + k] = ok ? arg : -1;
            weight[(size_t)n * top + k] = ok ? (by_logit ? 1.f / (1.f + expf(-z[arg])) : z[arg]) : 0.f;
            if (ok) taken[arg] = 1.f;
        }
        __syncwarp();
    }
    // renorm >= 0: the chosen scores are divided by their sum (+ renorm); then every weight times wscale
    if (lane == 0 && (renorm >= 0.f || wscale != 1.f)) {
        float sum = 0.f;
        for (int k = 0; k < top; ++k) sum += weight[(size_t)n * top + k];
        for (int k = 0; k < top; ++k) {
            float w = weight[(size_t)n * top + k];
            if (renorm >= 0.f) w = w / (sum + renorm);
            weight[(size_t)n * top + k] = w * wscale;
        }
    }
}

// A block takes RT rows, so that the 32-bit router matrix is read once for all of them.  Every thread takes a slice of
// the columns (four neighbouring ones at a time where the width allows) for eight router outputs at a time and all RT
// rows; the slices are added per warp by shuffles and across the warps through shared memory, in the same order
// whatever RT is: a row's logits do not depend on its neighbours in the block.  Then a warp per row scores and chooses.
template <typename T, int RT, bool VEC>
__global__ void __launch_bounds__(256)
moe_route_kernel(const T* __restrict__ h, const float* __restrict__ router, const float* __restrict__ correction,
                 const int* __restrict__ token_seq, int* __restrict__ choice, float* __restrict__ weight, int N, int D,
                 int n_out, int top, int scoring, float* __restrict__ logits, float renorm, float wscale) {
    pdl_enter();
    extern __shared__ float route_sm[];
    float* z_all = route_sm;                       // [RT][n_out] scores
    float* taken_all = z_all + RT * n_out;         // [RT][n_out] flags
    float* part = taken_all + RT * n_out;          // [warps][RT][n_out] partial sums
    const int n0 = blockIdx.x * RT, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const T* rows[RT];
#pragma unroll
    for (int r = 0; r < RT; ++r) rows[r] = h + (size_t)min(n0 + r, N - 1) * D;     // rows beyond the last: computed, not written
    // with `logits` the grid's second dimension cuts the router outputs into groups of eight: a block leaves its
    // group's logits there and moe_choose_kernel scores and chooses; without, one block does all of it
    const int e_lo = logits != nullptr ? blockIdx.y * 8 : 0, e_hi = logits != nullptr ? min(n_out, e_lo + 8) : n_out;
    for (int e0 = e_lo; e0 < e_hi; e0 += 8) {
        float s[RT][8];
#pragma unroll
        for (int r = 0; r < RT; ++r)
#pragma unroll
            for (int q = 0; q < 8; ++q) s[r][q] = 0.f;
        const int ne = min(8, n_out - e0);
        if constexpr (VEC) {
            for (int d = threadIdx.x * 4; d < D; d += blockDim.x * 4) {
                float4 x[RT];
#pragma unroll
                for (int r = 0; r < RT; ++r) x[r] = route_load4(rows[r] + d);
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    if (q < ne) {
                        const float4 w = *(const float4*)(router + (size_t)(e0 + q) * D + d);
#pragma unroll
                        for (int r = 0; r < RT; ++r)
                            s[r][q] = fmaf(x[r].w, w.w, fmaf(x[r].z, w.z, fmaf(x[r].y, w.y, fmaf(x[r].x, w.x, s[r][q]))));
                    }
                }
            }
        } else {
            for (int d = threadIdx.x; d < D; d += blockDim.x) {
                float x[RT];
#pragma unroll
                for (int r = 0; r < RT; ++r) x[r] = to_float(rows[r][d]);
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    if (q < ne) {
                        const float w = router[(size_t)(e0 + q) * D + d];
#pragma unroll
                        for (int r = 0; r < RT; ++r) s[r][q] = fmaf(x[r], w, s[r][q]);
                    }
                }
            }
        }
#pragma unroll
        for (int r = 0; r < RT; ++r)
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const float v = warp_sum(s[r][q]);
                if (lane == 0 && q < ne) part[(warp * RT + r) * n_out + e0 + q] = v;
            }
    }
    __syncthreads();
    if (logits != nullptr) {
        for (int i = threadIdx.x; i < RT * 8; i += blockDim.x) {
            const int r = i >> 3, e = e_lo + (i & 7);
            if (e >= e_hi || n0 + r >= N) continue;
            float v = 0.f;
            for (int w = 0; w < nwarps; ++w) v += part[(w * RT + r) * n_out + e];
            logits[(size_t)(n0 + r) * n_out + e] = v;
        }
        return;
    }
    for (int i = threadIdx.x; i < RT * n_out; i += blockDim.x) {
        float v = 0.f;
        for (int w = 0; w < nwarps; ++w) v += part[w * RT * n_out + i];
        z_all[i] = v;
        taken_all[i] = 0.f;
    }
    __syncthreads();
    if (warp >= RT) return;
    const int n = n0 + warp;
    if (n >= N) return;
    route_choose(z_all + warp * n_out, taken_all + warp * n_out, correction, token_seq, choice, weight, n, n_out, top, scoring,
                 lane, renorm, wscale);
}

// A warp per row: logits [N][n_out] from moe_route_kernel's blocks -> scores, the `top` largest, their weights.
__global__ void __launch_bounds__(128)
moe_choose_kernel(const float* __restrict__ logits, const float* __restrict__ correction, const int* __restrict__ token_seq,
                  int* __restrict__ choice, float* __restrict__ weight, int N, int n_out, int top, int scoring,
                  float renorm, float wscale) {
    pdl_enter();
    extern __shared__ float route_sm[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int n = blockIdx.x * nwarps + warp;
    if (n >= N) return;
    float* z = route_sm + (size_t)warp * 2 * n_out;
    float* taken = z + n_out;
    for (int e = lane; e < n_out; e += 32) {
        z[e] = logits[(size_t)n * n_out + e];
        taken[e] = 0.f;
    }
    __syncwarp();
    route_choose(z, taken, correction, token_seq, choice, weight, n, n_out, top, scoring, lane, renorm, wscale);
}

// One block.  listed: [cap] pair ids (row * top + choice) expert by expert, -1 where a tile is padded;
// tile_expert: [max_tiles], -1 beyond the real tiles.
__global__ void moe_align_kernel(const int* __restrict__ choice, int n_pairs, int n_experts, int* __restrict__ listed,
                                 int cap, int* __restrict__ tile_expert, int max_tiles) {
    pdl_enter();
    extern __shared__ int sh[];                // count[n_experts], start[n_experts + 1], cursor[n_experts]
    int* count = sh;
    int* start = count + n_experts;
    int* cursor = start + n_experts + 1;
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) count[e] = cursor[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
        const int e = choice[i];
        if (e >= 0 && e < n_experts) atomicAdd(&count[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < n_experts; ++e) {
            start[e] = at;
            const int tiles = (count[e] + kTile - 1) / kTile;
            for (int t = 0; t < tiles; ++t)
                if (at / kTile + t < max_tiles) tile_expert[at / kTile + t] = e;
            at += tiles * kTile;
        }
        start[n_experts] = at;
        for (int t = at / kTile; t < max_tiles; ++t) tile_expert[t] = -1;
    }
    __syncthreads();
    const int used = min(start[n_experts], cap);
    for (int i = threadIdx.x; i < used; i += blockDim.x) listed[i] = -1;
    __syncthreads();
    for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
        const int e = choice[i];
        if (e >= 0 && e < n_experts) {
            const int p = start[e] + atomicAdd(&cursor[e], 1);
            if (p < cap) listed[p] = i;
        }
    }
}

// y[listed position][F] = act(gate, up) of the listed rows; W: [experts][2F][D], gate rows then up rows.
template <typename T>
__global__ void __launch_bounds__(256)
moe_gate_up_kernel(const T* __restrict__ h, const T* __restrict__ W, const int* __restrict__ listed,
                   const int* __restrict__ tile_expert, T* __restrict__ y, int D, int F, int top, float limit,
                   float alpha, float up_shift, const float* __restrict__ in_weight) {
    pdl_enter();
    constexpr int BK = 16;
    __shared__ float As[BK][kTile + 4];
    __shared__ float Gs[BK][kTile + 4];
    __shared__ float Us[BK][kTile + 4];
    __shared__ int rows[kTile];
    const int tile = blockIdx.y, e = tile_expert[tile];
    if (e < 0) return;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4, n0 = blockIdx.x * kTile;
    if (threadIdx.x < kTile) {
        const int id = listed[tile * kTile + threadIdx.x];
        rows[threadIdx.x] = id >= 0 ? id / top : -1;
    }
    __syncthreads();
    const int warp_row0 = (threadIdx.x >> 5) * 8;          // a warp's threads hold rows warp_row0 .. +7
    bool busy = false;
    for (int i = 0; i < 8; ++i) busy = busy || rows[warp_row0 + i] >= 0;
    const T* Wg = W + (size_t)e * 2 * F * D;
    const T* Wu = Wg + (size_t)F * D;
    float acc_g[4][4] = {}, acc_u[4][4] = {};
    for (int k0 = 0; k0 < D; k0 += BK) {
        for (int x = threadIdx.x; x < kTile * BK; x += 256) {
            const int r = x >> 4, kk = x & 15, k = k0 + kk, n = n0 + r;
            const int src = rows[r];
            As[kk][r] = (src >= 0 && k < D) ? to_float(h[(size_t)src * D + k]) : 0.f;
            const bool in = n < F && k < D;
            Gs[kk][r] = in ? to_float(Wg[(size_t)n * D + k]) : 0.f;
            Us[kk][r] = in ? to_float(Wu[(size_t)n * D + k]) : 0.f;
        }
        __syncthreads();
        if (busy) {
#pragma unroll
            for (int kk = 0; kk < BK; ++kk) {
                float a[4], g[4], u[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    g[j] = Gs[kk][tx * 4 + j];
                    u[j] = Us[kk][tx * 4 + j];
                }
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        acc_g[i][j] = fmaf(a[i], g[j], acc_g[i][j]);
                        acc_u[i][j] = fmaf(a[i], u[j], acc_u[i][j]);
                    }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = ty * 4 + i;
        if (rows[r] < 0) continue;
        const float wt = in_weight ? in_weight[listed[tile * kTile + r]] : 1.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= F) continue;
            float g = acc_g[i][j] * wt, u = acc_u[i][j] * wt;
            if (limit > 0.f) {
                g = fminf(g, limit);
                u = fminf(fmaxf(u, -limit), limit);
            }
            const float v = g / (1.f + expf(-alpha * g)) * (u + up_shift);
            y[(size_t)(tile * kTile + r) * F + n] = from_float<T>(v);
        }
    }
}

// pair_out[pair id][D] = weight[pair id] * (W_down[e] . y[listed position]); W: [experts][D][F].
template <typename T>
__global__ void __launch_bounds__(256)
moe_down_kernel(const T* __restrict__ y, const T* __restrict__ W, const int* __restrict__ listed,
                const int* __restrict__ tile_expert, const float* __restrict__ weight, float* __restrict__ pair_out,
                int D, int F) {
    pdl_enter();
    constexpr int BK = 16;
    __shared__ float As[BK][kTile + 4];
    __shared__ float Ws[BK][kTile + 4];
    __shared__ int ids[kTile];
    const int tile = blockIdx.y, e = tile_expert[tile];
    if (e < 0) return;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4, n0 = blockIdx.x * kTile;
    if (threadIdx.x < kTile) ids[threadIdx.x] = listed[tile * kTile + threadIdx.x];
    __syncthreads();
    const int warp_row0 = (threadIdx.x >> 5) * 8;
    bool busy = false;
    for (int i = 0; i < 8; ++i) busy = busy || ids[warp_row0 + i] >= 0;
    const T* Wd = W + (size_t)e * D * F;
    const T* A = y + (size_t)tile * kTile * F;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < F; k0 += BK) {
        for (int x = threadIdx.x; x < kTile * BK; x += 256) {
            const int r = x >> 4, kk = x & 15, k = k0 + kk, n = n0 + r;
            As[kk][r] = (ids[r] >= 0 && k < F) ? to_float(A[(size_t)r * F + k]) : 0.f;
            Ws[kk][r] = (n < D && k < F) ? to_float(Wd[(size_t)n * F + k]) : 0.f;
        }
        __syncthreads();
        if (busy) {
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
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int id = ids[ty * 4 + i];
        if (id < 0) continue;
        const float wt = weight ? weight[id] : 1.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < D) pair_out[(size_t)id * D + n] = acc[i][j] * wt;
        }
    }
}

// ---- the bfloat16 products on the tensor cores ----------------------------------------------------
// Tiles of 64 rows x 64 output features, K in steps of 64 through a ring of kStages shared-memory stages
// filled by 16-byte asynchronous copies; rows of 128 bytes with their 16-byte groups XOR-permuted by the
// row so that ldmatrix reads without bank conflicts; 8 warps as 4 (rows) x 2 (features), m16n8k16 MMAs with
// 32-bit accumulators.  A warp whose 16 rows are all padding issues no MMA (a decode step's tiles hold a
// few rows each: the launch is then bound by the weights it streams).  K and the row strides must be
// multiples of 8 (16-byte rows); other sizes take the kernels above.
__global__ void __launch_bounds__(256)
moe_gate_up_tc_kernel(const bf16* __restrict__ h, const bf16* __restrict__ W, const int* __restrict__ listed,
                      const int* __restrict__ tile_expert, bf16* __restrict__ y, int D, int F, int top, float limit,
                      float alpha, float up_shift, const float* __restrict__ in_weight) {
    pdl_enter();
    extern __shared__ __align__(128) unsigned char raw[];
    bf16* smem = reinterpret_cast<bf16*>(raw);
    __shared__ int rows[kTile];
    const int tile = blockIdx.y, e = tile_expert[tile];
    if (e < 0) return;
    const int n0 = blockIdx.x * kTile, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x < kTile) {
        const int id = listed[tile * kTile + threadIdx.x];
        rows[threadIdx.x] = id >= 0 ? id / top : -1;
    }
    __syncthreads();
    const int warp_m = warp & 3, warp_n = warp >> 2;
    bool busy = false;
    for (int i = 0; i < 16; ++i) busy = busy || rows[warp_m * 16 + i] >= 0;
    float acc[2][4][4] = {};
    const bf16* We = W + (size_t)e * 2 * F * D;
    tc_mainloop<2>(smem, [&](int r) { return rows[r] >= 0 ? h + (size_t)rows[r] * D : (const bf16*)nullptr; }, We, F, n0,
                   (size_t)F * D, D, busy, acc);
    if (!busy) return;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
        const int n = n0 + warp_n * 32 + nt * 8 + (lane & 3) * 2;
        if (n >= F) continue;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = warp_m * 16 + (lane >> 2) + half * 8;
            if (rows[r] < 0) continue;
            const float wt = in_weight ? in_weight[listed[tile * kTile + r]] : 1.f;
            float v[2];
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                float g = acc[0][nt][half * 2 + c] * wt, u = acc[1][nt][half * 2 + c] * wt;
                if (limit > 0.f) {
                    g = fminf(g, limit);
                    u = fminf(fmaxf(u, -limit), limit);
                }
                v[c] = g / (1.f + expf(-alpha * g)) * (u + up_shift);
            }
            *reinterpret_cast<uint32_t*>(y + (size_t)(tile * kTile + r) * F + n) = pack_bf16(v[0], v[1]);
        }
    }
}

__global__ void __launch_bounds__(256)
moe_down_tc_kernel(const bf16* __restrict__ y, const bf16* __restrict__ W, const int* __restrict__ listed,
                   const int* __restrict__ tile_expert, const float* __restrict__ weight, float* __restrict__ pair_out,
                   int D, int F) {
    pdl_enter();
    extern __shared__ __align__(128) unsigned char raw[];
    bf16* smem = reinterpret_cast<bf16*>(raw);
    __shared__ int ids[kTile];
    const int tile = blockIdx.y, e = tile_expert[tile];
    if (e < 0) return;
    const int n0 = blockIdx.x * kTile, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x < kTile) ids[threadIdx.x] = listed[tile * kTile + threadIdx.x];
    __syncthreads();
    const int warp_m = warp & 3, warp_n = warp >> 2;
    bool busy = false;
    for (int i = 0; i < 16; ++i) busy = busy || ids[warp_m * 16 + i] >= 0;
    float acc[1][4][4] = {};
    const bf16* A = y + (size_t)tile * kTile * F;
    tc_mainloop<1>(smem, [&](int r) { return ids[r] >= 0 ? A + (size_t)r * F : (const bf16*)nullptr; },
                   W + (size_t)e * D * F, D, n0, 0, F, busy, acc);
    if (!busy) return;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int id = ids[warp_m * 16 + (lane >> 2) + half * 8];
        if (id < 0) continue;
        const float wt = weight ? weight[id] : 1.f;
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            const int n = n0 + warp_n * 32 + nt * 8 + (lane & 3) * 2;
            if (n < D)
                *reinterpret_cast<float2*>(pair_out + (size_t)id * D + n) =
                    make_float2(acc[0][nt][half * 2] * wt, acc[0][nt][half * 2 + 1] * wt);
        }
    }
}

// ---- a handful of rows (decoding at small batch) ---------------------------------------------------
// With a few (row, choice) pairs a tile of 64 rows is nearly empty and there are too few tiles to fill the GPU.
// These kernels take the pairs as they are: a block per (pair, 8 * QF output features), a warp per QF features, every
// lane 16 bytes of each of its weight rows at a time against the activation row in shared memory.  A warp walks its
// QF features' rows together, so that 2 QF (gate and up) or QF independent 16-byte loads are under way per lane and
// step, and the loads of several steps are issued together (16 a lane): the launch is bound by the weights it
// streams, and a lone load per step leaves the memory idle.  QF is the largest of 4, 2, 1 that still gives two
// blocks to an SM (fewer blocks of more features leave SMs idle or with twice the work of others; more blocks of
// fewer features read the activation row more often).  The weights of an expert that several pairs chose are read
// again from L2.  bfloat16, K a multiple of 8.
__device__ __forceinline__ float dot8(const uint4& a, const uint4& b) {
    const uint32_t x[4] = {a.x, a.y, a.z, a.w}, y[4] = {b.x, b.y, b.z, b.w};
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        s = fmaf(__uint_as_float(x[i] << 16), __uint_as_float(y[i] << 16), s);
        s = fmaf(__uint_as_float(x[i] & 0xffff0000u), __uint_as_float(y[i] & 0xffff0000u), s);
    }
    return s;
}

// y[pair][F] = act(gate, up) of row pair / top under expert choice[pair]
template <int QF>
__global__ void __launch_bounds__(256)
moe_gate_up_few_kernel(const bf16* __restrict__ h, const bf16* __restrict__ W, const int* __restrict__ choice,
                       bf16* __restrict__ y, int D, int F, int top, int n_experts, float limit, float alpha,
                       float up_shift, const float* __restrict__ in_weight) {
    pdl_enter();
    extern __shared__ __align__(128) unsigned char raw[];
    uint4* row = reinterpret_cast<uint4*>(raw);                 // the activation row, 8 numbers a group
    const int pair = blockIdx.y, e = choice[pair];
    if (e < 0 || e >= n_experts) return;
    const int groups = D >> 3, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint4* src = reinterpret_cast<const uint4*>(h + (size_t)(pair / top) * D);
    for (int g = threadIdx.x; g < groups; g += 256) row[g] = src[g];
    __syncthreads();
    const bf16* Wg = W + (size_t)e * 2 * F * D;
    const int f0 = (blockIdx.x * 8 + warp) * QF;
    if (f0 >= F) return;
    const uint4* g_row[QF];
    const uint4* u_row[QF];
#pragma unroll
    for (int q = 0; q < QF; ++q) {
        const int f = min(f0 + q, F - 1);                       // a feature beyond the last: read the last again, store nothing
        g_row[q] = reinterpret_cast<const uint4*>(Wg + (size_t)f * D);
        u_row[q] = reinterpret_cast<const uint4*>(Wg + (size_t)(F + f) * D);
    }
    float sg[QF], su[QF];
#pragma unroll
    for (int q = 0; q < QF; ++q) sg[q] = su[q] = 0.f;
    constexpr int U = 8 / QF;                                   // steps whose loads are issued together: 16 loads a lane
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    for (int g0 = lane; g0 < groups; g0 += 32 * U) {
        uint4 wg[U][QF], wu[U][QF];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int g = g0 + 32 * u;
#pragma unroll
            for (int q = 0; q < QF; ++q) {
                wg[u][q] = g < groups ? __ldg(g_row[q] + g) : zero;
                wu[u][q] = g < groups ? __ldg(u_row[q] + g) : zero;
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int g = g0 + 32 * u;
            if (g >= groups) break;
            const uint4 x = row[g];
#pragma unroll
            for (int q = 0; q < QF; ++q) {
                sg[q] += dot8(x, wg[u][q]);
                su[q] += dot8(x, wu[u][q]);
            }
        }
    }
    const float wt = in_weight ? in_weight[pair] : 1.f;
#pragma unroll
    for (int q = 0; q < QF; ++q) {
        float a = warp_sum(sg[q]) * wt, b = warp_sum(su[q]) * wt;
        if (lane == 0 && f0 + q < F) {
            if (limit > 0.f) {
                a = fminf(a, limit);
                b = fminf(fmaxf(b, -limit), limit);
            }
            y[(size_t)pair * F + f0 + q] = from_float<bf16>(a / (1.f + expf(-alpha * a)) * (b + up_shift));
        }
    }
}

// pair_out[pair][D] = weight[pair] * (W_down[e] . y[pair])
template <int QF>
__global__ void __launch_bounds__(256)
moe_down_few_kernel(const bf16* __restrict__ y, const bf16* __restrict__ W, const int* __restrict__ choice,
                    const float* __restrict__ weight, float* __restrict__ pair_out, int D, int F, int n_experts) {
    pdl_enter();
    extern __shared__ __align__(128) unsigned char raw[];
    uint4* row = reinterpret_cast<uint4*>(raw);
    const int pair = blockIdx.y, e = choice[pair];
    if (e < 0 || e >= n_experts) return;
    const int groups = F >> 3, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint4* src = reinterpret_cast<const uint4*>(y + (size_t)pair * F);
    for (int g = threadIdx.x; g < groups; g += 256) row[g] = src[g];
    __syncthreads();
    const bf16* Wd = W + (size_t)e * D * F;
    const float wt = weight ? weight[pair] : 1.f;
    const int n0 = (blockIdx.x * 8 + warp) * QF;
    if (n0 >= D) return;
    const uint4* w_row[QF];
#pragma unroll
    for (int q = 0; q < QF; ++q) w_row[q] = reinterpret_cast<const uint4*>(Wd + (size_t)min(n0 + q, D - 1) * F);
    float s[QF];
#pragma unroll
    for (int q = 0; q < QF; ++q) s[q] = 0.f;
    constexpr int U = 16 / QF;                                  // steps whose loads are issued together: 16 loads a lane
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    for (int g0 = lane; g0 < groups; g0 += 32 * U) {
        uint4 w[U][QF];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int g = g0 + 32 * u;
#pragma unroll
            for (int q = 0; q < QF; ++q) w[u][q] = g < groups ? __ldg(w_row[q] + g) : zero;
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int g = g0 + 32 * u;
            if (g >= groups) break;
            const uint4 x = row[g];
#pragma unroll
            for (int q = 0; q < QF; ++q) s[q] += dot8(x, w[u][q]);
        }
    }
#pragma unroll
    for (int q = 0; q < QF; ++q) {
        const float t = warp_sum(s[q]);
        if (lane == 0 && n0 + q < D) pair_out[(size_t)pair * D + n0 + q] = t * wt;
    }
}

// A block per row and per 256 * VEC columns: the chosen pairs' rows are independent loads, so a row of any width
// costs one round of them.  VEC = 4 where the width and the addresses allow 16-byte accesses.
template <typename T, int VEC>
__global__ void __launch_bounds__(256)
moe_combine_kernel(const float* __restrict__ pair_out, const int* __restrict__ choice, const float* __restrict__ weight,
                   const T* __restrict__ h, float* __restrict__ out, int D, int top, int n_experts,
                   const T* __restrict__ extra) {
    pdl_enter();
    const int n = blockIdx.x;
    const int d = (blockIdx.y * 256 + threadIdx.x) * VEC;
    if (d >= D) return;
    float s[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) s[i] = extra ? to_float(extra[(size_t)n * D + d + i]) : 0.f;
#pragma unroll 4
    for (int k = 0; k < top; ++k) {
        const size_t id = (size_t)n * top + k;
        const int e = choice[id];
        if (e < 0) continue;
        if (e < n_experts) {
            if constexpr (VEC == 4) {
                const float4 p = *(const float4*)(pair_out + id * D + d);
                s[0] += p.x; s[1] += p.y; s[2] += p.z; s[3] += p.w;
            } else {
                s[0] += pair_out[id * D + d];
            }
        } else {
            const float w = weight[id];
#pragma unroll
            for (int i = 0; i < VEC; ++i) s[i] = fmaf(w, to_float(h[(size_t)n * D + d + i]), s[i]);
        }
    }
    if constexpr (VEC == 4) *(float4*)(out + (size_t)n * D + d) = make_float4(s[0], s[1], s[2], s[3]);
    else out[(size_t)n * D + d] = s[0];
}

}  // namespace hos

static int sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (n <= 0) n = 148;
    }
    return n;
}

using namespace hos;

extern "C" const char* hos_last_error() { return error_buffer(); }

extern "C" int hos_moe_tile_rows() { return kTile; }

extern "C" int hos_moe_route(const void* h, int dtype, const float* router, const float* correction,
                             const int* token_seq, int* choice, float* weight, int N, int D, int n_out, int top,
                             int scoring, float* logits, float renorm, float wscale, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (top <= 0 || top > n_out) HOS_REFUSE("moe_route: %d of %d router outputs cannot be chosen", top, n_out);
    // rows to a block: as many as pay (the router matrix is read once per block) and as shared memory holds
    int rt = N >= 1024 ? 8 : N >= 16 ? 4 : 1;
    auto smem_of = [&](int r) { return (size_t)(2 + 8) * r * n_out * sizeof(float); };   // scores, flags, a partial sum per warp
    while (rt > 1 && smem_of(rt) > 48 * 1024) rt = rt == 8 ? 4 : 1;
    const size_t smem = smem_of(rt);
    if (smem > 48 * 1024) HOS_REFUSE("moe_route: %d router outputs are more than a block's shared memory holds", n_out);
    if (dtype != kBF16 && dtype != kF32) HOS_REFUSE("moe_route: unknown dtype %d", dtype);
    const bool vec = D % 4 == 0 && (uintptr_t)router % 16 == 0 && (uintptr_t)h % (dtype == kBF16 ? 8 : 16) == 0;
    const unsigned blocks = (unsigned)((N + rt - 1) / rt);
    // few blocks and more than eight outputs: the outputs' groups of eight go to blocks of their own (grid.y) and a
    // second launch chooses; the caller then gives `logits` [N][n_out]
    if (blocks >= 296u || n_out <= 8) logits = nullptr;
    const unsigned groups = logits != nullptr ? (unsigned)((n_out + 7) / 8) : 1u;
#define HOS_ROUTE(T, RT, VEC)                                                                                        \
    launch_pdl(moe_route_kernel<T, RT, VEC>, dim3(blocks, groups), dim3(256), smem, stream, (const T*)h, router,     \
               correction, token_seq, choice, weight, N, D, n_out, top, scoring, logits, renorm, wscale)
#define HOS_ROUTE_V(T, RT)                                                                                           \
    do {                                                                                                             \
        if (vec) HOS_ROUTE(T, RT, true);                                                                             \
        else HOS_ROUTE(T, RT, false);                                                                                \
    } while (0)
#define HOS_ROUTE_R(T)                                                                                               \
    do {                                                                                                             \
        if (rt == 8) HOS_ROUTE_V(T, 8);                                                                              \
        else if (rt == 4) HOS_ROUTE_V(T, 4);                                                                         \
        else HOS_ROUTE_V(T, 1);                                                                                      \
    } while (0)
    if (dtype == kBF16) HOS_ROUTE_R(bf16);
    else HOS_ROUTE_R(float);
#undef HOS_ROUTE_R
#undef HOS_ROUTE_V
#undef HOS_ROUTE
    if (logits != nullptr) {
        const size_t csmem = (size_t)4 * 2 * n_out * sizeof(float);
        if (csmem > 48 * 1024) HOS_REFUSE("moe_route: %d router outputs are more than a block's shared memory holds", n_out);
        launch_pdl(moe_choose_kernel, dim3((N + 3) / 4), dim3(128), csmem, stream, (const float*)logits, correction, token_seq,
                   choice, weight, N, n_out, top, scoring, renorm, wscale);
    }
    return check_launch("moe_route");
}

extern "C" int hos_moe_align(const int* choice, int n_pairs, int n_experts, int* listed, int cap, int* tile_expert,
                             int max_tiles, cudaStream_t stream) {
    if (n_pairs <= 0) return 0;
    const size_t smem = (size_t)(3 * n_experts + 1) * sizeof(int);
    if (smem > 48 * 1024) HOS_REFUSE("moe_align: %d experts are more than a block's shared memory holds", n_experts);
    launch_pdl(moe_align_kernel, dim3(1), dim3(1024), smem, stream, choice, n_pairs, n_experts, listed, cap, tile_expert,
               max_tiles);
    return check_launch("moe_align");
}

extern "C" int hos_moe_gate_up(const void* h, const void* W, int dtype, const int* listed, const int* tile_expert,
                               void* y, int max_tiles, int D, int F, int top, float limit, float alpha, float up_shift,
                               const float* in_weight, cudaStream_t stream) {
    if (max_tiles <= 0) return 0;
    dim3 grid((F + kTile - 1) / kTile, max_tiles);
    if (grid.y > 65535) HOS_REFUSE("moe_gate_up: %d tiles are more than one launch takes", max_tiles);
    if (dtype == kBF16 && D % 8 == 0 && F % 8 == 0 && ((uintptr_t)h | (uintptr_t)W | (uintptr_t)y) % 16 == 0) {
        static bool set = false;
        if (!set) {
            cudaFuncSetAttribute(moe_gate_up_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TcTile<2>::kSmemBytes);
            set = true;
        }
        launch_pdl(moe_gate_up_tc_kernel, grid, dim3(256), (size_t)TcTile<2>::kSmemBytes, stream, (const bf16*)h,
                   (const bf16*)W, listed, tile_expert, (bf16*)y, D, F, top, limit, alpha, up_shift, in_weight);
    } else if (dtype == kBF16)
        launch_pdl(moe_gate_up_kernel<bf16>, grid, dim3(256), 0, stream, (const bf16*)h, (const bf16*)W, listed, tile_expert,
                   (bf16*)y, D, F, top, limit, alpha, up_shift, in_weight);
    else if (dtype == kF32)
        launch_pdl(moe_gate_up_kernel<float>, grid, dim3(256), 0, stream, (const float*)h, (const float*)W, listed,
                   tile_expert, (float*)y, D, F, top, limit, alpha, up_shift, in_weight);
    else
        HOS_REFUSE("moe_gate_up: unknown dtype %d", dtype);
    return check_launch("moe_gate_up");
}

extern "C" int hos_moe_down(const void* y, const void* W, int dtype, const int* listed, const int* tile_expert,
                            const float* weight, float* pair_out, int max_tiles, int D, int F, cudaStream_t stream) {
    if (max_tiles <= 0) return 0;
    dim3 grid((D + kTile - 1) / kTile, max_tiles);
    if (grid.y > 65535) HOS_REFUSE("moe_down: %d tiles are more than one launch takes", max_tiles);
    if (dtype == kBF16 && D % 8 == 0 && F % 8 == 0 && ((uintptr_t)y | (uintptr_t)W | (uintptr_t)pair_out) % 16 == 0) {
        static bool set = false;
        if (!set) {
            cudaFuncSetAttribute(moe_down_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TcTile<1>::kSmemBytes);
            set = true;
        }
        launch_pdl(moe_down_tc_kernel, grid, dim3(256), (size_t)TcTile<1>::kSmemBytes, stream, (const bf16*)y,
                   (const bf16*)W, listed, tile_expert, weight, pair_out, D, F);
    } else if (dtype == kBF16)
        launch_pdl(moe_down_kernel<bf16>, grid, dim3(256), 0, stream, (const bf16*)y, (const bf16*)W, listed, tile_expert,
                   weight, pair_out, D, F);
    else if (dtype == kF32)
        launch_pdl(moe_down_kernel<float>, grid, dim3(256), 0, stream, (const float*)y, (const float*)W, listed, tile_expert,
                   weight, pair_out, D, F);
    else
        HOS_REFUSE("moe_down: unknown dtype %d", dtype);
    return check_launch("moe_down");
}

extern "C" int hos_moe_combine(const float* pair_out, const int* choice, const float* weight, const void* h, int dtype,
                               float* out, int N, int D, int top, int n_experts, const void* extra, cudaStream_t stream) {
    if (N <= 0) return 0;
    const bool vec = D % 4 == 0 && ((uintptr_t)pair_out | (uintptr_t)out) % 16 == 0;
    const dim3 grid((unsigned)N, (unsigned)((D + (vec ? 1024 : 256) - 1) / (vec ? 1024 : 256)));
    if (grid.y > 65535) HOS_REFUSE("moe_combine: rows of %d numbers are more than one launch takes", D);
#define HOS_COMBINE(T, VEC)                                                                                          \
    launch_pdl(moe_combine_kernel<T, VEC>, grid, dim3(256), 0, stream, pair_out, choice, weight, (const T*)h, out, D, top, \
               n_experts, (const T*)extra)
    if (dtype == kBF16) {
        if (vec) HOS_COMBINE(bf16, 4);
        else HOS_COMBINE(bf16, 1);
    } else if (dtype == kF32) {
        if (vec) HOS_COMBINE(float, 4);
        else HOS_COMBINE(float, 1);
    } else
        HOS_REFUSE("moe_combine: unknown dtype %d", dtype);
#undef HOS_COMBINE
    return check_launch("moe_combine");
}

// The same two products for a handful of pairs (see the kernels): y is [pairs][F] by pair id.  Returns 1 (and
// launches nothing) where the sizes are not the kernels' (K no multiple of 8, rows that do not fit shared memory).
extern "C" int hos_moe_gate_up_few(const void* h, const void* W, const int* choice, void* y, int n_pairs, int D, int F,
                                   int top, int n_experts, float limit, float alpha, float up_shift, const float* in_weight,
                                   cudaStream_t stream) {
    if (n_pairs <= 0) return 0;
    if (D % 8 || F % 8 || D * 2 > 96 * 1024 || ((uintptr_t)h | (uintptr_t)W | (uintptr_t)y) % 16) return 1;
    const long long want = 2LL * sm_count();
    const int qf = (long long)((F + 31) / 32) * n_pairs >= want ? 4 : (long long)((F + 15) / 16) * n_pairs >= want ? 2 : 1;
#define HOS_GU_FEW(QF)                                                                                               \
    do {                                                                                                             \
        if (D * 2 > 48 * 1024)                                                                                       \
            cudaFuncSetAttribute(moe_gate_up_few_kernel<QF>, cudaFuncAttributeMaxDynamicSharedMemorySize, D * 2);    \
        launch_pdl(moe_gate_up_few_kernel<QF>, dim3((F + 8 * QF - 1) / (8 * QF), n_pairs), dim3(256), (size_t)D * 2, \
                   stream, (const bf16*)h, (const bf16*)W, choice, (bf16*)y, D, F, top, n_experts, limit, alpha,     \
                   up_shift, in_weight);                                                                             \
    } while (0)
    if (qf == 4) HOS_GU_FEW(4);
    else if (qf == 2) HOS_GU_FEW(2);
    else HOS_GU_FEW(1);
#undef HOS_GU_FEW
    return check_launch("moe_gate_up_few");
}

extern "C" int hos_moe_down_few(const void* y, const void* W, const int* choice, const float* weight, float* pair_out,
                                int n_pairs, int D, int F, int n_experts, cudaStream_t stream) {
    if (n_pairs <= 0) return 0;
    if (D % 8 || F % 8 || F * 2 > 96 * 1024 || ((uintptr_t)y | (uintptr_t)W) % 16) return 1;
    const long long want = 2LL * sm_count();
    const int qf = (long long)((D + 31) / 32) * n_pairs >= want ? 4 : (long long)((D + 15) / 16) * n_pairs >= want ? 2 : 1;
#define HOS_DOWN_FEW(QF)                                                                                             \
    do {                                                                                                             \
        if (F * 2 > 48 * 1024)                                                                                       \
            cudaFuncSetAttribute(moe_down_few_kernel<QF>, cudaFuncAttributeMaxDynamicSharedMemorySize, F * 2);       \
        launch_pdl(moe_down_few_kernel<QF>, dim3((D + 8 * QF - 1) / (8 * QF), n_pairs), dim3(256), (size_t)F * 2,    \
                   stream, (const bf16*)y, (const bf16*)W, choice, weight, pair_out, D, F, n_experts);               \
    } while (0)
    if (qf == 4) HOS_DOWN_FEW(4);
    else if (qf == 2) HOS_DOWN_FEW(2);
    else HOS_DOWN_FEW(1);
#undef HOS_DOWN_FEW
    return check_launch("moe_down_few");
}
