// A feed-forward of routed experts: router, grouping of the tokens by expert, the experts' two
// matrix products over the groups, and the weighted sum back into the residual stream.
//
//   route:   z = W_r h (32-bit), the `top` largest z choose experts (ties: the lower index), their
//            weights are softmax over the chosen z alone; optionally g = sigmoid(w_g . h), one number
//            per token (the gate of an expert that every token uses).
//   group:   entry (token, k) -> a slot; the slots of one expert are contiguous and in entry order.
//   experts: H[slot] = silu(W_gate[e] h) * (W_up[e] h);  Y[slot] = weight[slot] * W_down[e] H[slot]  (32-bit)
//   combine: x[token] += sum_k Y[slot of (token, k)], k in order: the same sum whatever the grouping.
//
// Nothing here depends on the host knowing how many tokens an expert got: grids are sized for the
// worst case and blocks without work leave at once, so the whole part can sit in a CUDA graph.  Every
// output element sums its terms in one fixed order (k = 0, 1, 2, ...), whatever else is in the batch.
#include <math.h>

#include "common.cuh"

MG_GUARD_DECLARE(moe)

namespace {

// ---- router ------------------------------------------------------------------------------------
// One CTA per token: its warps share the experts (and the gate, as one more row of weights), a lane
// sums every 32nd group of four features in a fixed order, so a token's logits depend on nothing
// but the token.  Warp 0 then picks the `top` largest one after the other.
constexpr int ROUTE_WARPS = 8;

template <typename T>
__device__ __forceinline__ float route_dot(const T* __restrict__ row, const float* __restrict__ wr, int width, int lane,
                                           bool vec) {
    float dot = 0.f;
    if (vec) {
#pragma unroll 4
        for (int c = lane * 4; c < width; c += 128) {
            const float4 wv = *reinterpret_cast<const float4*>(wr + c);
            dot = fmaf(to_float(row[c]), wv.x, dot);
            dot = fmaf(to_float(row[c + 1]), wv.y, dot);
            dot = fmaf(to_float(row[c + 2]), wv.z, dot);
            dot = fmaf(to_float(row[c + 3]), wv.w, dot);
        }
    } else {
        for (int c = lane; c < width; c += 32) dot = fmaf(to_float(row[c]), wr[c], dot);
    }
    return warp_sum(dot);
}

template <typename T>
__global__ void __launch_bounds__(32 * ROUTE_WARPS)
moe_route_kernel(const T* __restrict__ h, const float* __restrict__ w_router, const float* __restrict__ w_gate,
                 const int* __restrict__ positions, int* __restrict__ ids, float* __restrict__ weights,
                 float* __restrict__ gate, int n_tokens, int width, int n_experts, int top) {
    extern __shared__ float z[];                           // [n_experts]
    pdl_trigger();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int token = blockIdx.x;
    if (positions != nullptr && positions[token] < 0) {    // padding of a fixed-size batch: no expert
        for (int k = threadIdx.x; k < top; k += blockDim.x) {
            ids[(size_t)token * top + k] = -1;
            weights[(size_t)token * top + k] = 0.f;
        }
        if (gate != nullptr && threadIdx.x == 0) gate[token] = 0.f;
        return;
    }
    const T* row = h + (size_t)token * width;
    const bool vec = width % 4 == 0 && ((uintptr_t)w_router % 16 == 0) && (w_gate == nullptr || (uintptr_t)w_gate % 16 == 0);
    const int rows = n_experts + (gate != nullptr ? 1 : 0);
    for (int e = warp; e < rows; e += ROUTE_WARPS) {
        const float dot = route_dot(row, e < n_experts ? w_router + (size_t)e * width : w_gate, width, lane, vec);
        if (lane == 0) {
            if (e < n_experts) z[e] = dot;
            else gate[token] = 1.0f / (1.0f + expf(-dot));
        }
    }
    __syncthreads();
    if (warp != 0) return;
    // the `top` largest, one after the other; every lane looks at a share of the experts
    float z_max = 0.f, sum = 0.f;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int best_e = 0x7fffffff;
        for (int e = lane; e < n_experts; e += 32) {
            const float v = z[e];
            if (v > best || (v == best && e < best_e)) best = v, best_e = e;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (ov > best || (ov == best && oe < best_e)) best = ov, best_e = oe;
        }
        if (best_e >= n_experts) best_e = k;               // logits that are not numbers: still a valid choice
        if (k == 0) z_max = best;
        const float p = expf(best - z_max);
        sum += p;
        if (lane == 0) {
            ids[(size_t)token * top + k] = best_e;
            weights[(size_t)token * top + k] = p;
            z[best_e] = -INFINITY;
        }
        __syncwarp();
    }
    const float inv = 1.0f / sum;
    for (int k = lane; k < top; k += 32) weights[(size_t)token * top + k] *= inv;
}

// ---- router with scores per expert, a correction for the choice, and groups --------------------------
// scoring 1: s = sigmoid(z), weights = scale * s of the chosen experts (not renormalised);
// scoring 0: s = z, weights = scale * softmax over the chosen z.
// Choice scores c = s + correction (correction may be null).  With n_groups > 0 the experts form n_groups equal
// groups of neighbours; a group's score is the sum of its two largest c (of its one c, if it has one expert),
// and only experts of the `keep` best groups can be chosen.  Ties go to the lower index.
__device__ __forceinline__ void warp_argmax(float& best, int& best_i) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (ov > best || (ov == best && oi < best_i)) best = ov, best_i = oi;
    }
}

template <typename T>
__global__ void __launch_bounds__(32 * ROUTE_WARPS)
moe_route_scored_kernel(const T* __restrict__ h, const float* __restrict__ w_router, const float* __restrict__ w_gate,
                        const float* __restrict__ correction, const int* __restrict__ positions, int* __restrict__ ids,
                        float* __restrict__ weights, float* __restrict__ gate, int n_tokens, int width, int n_experts,
                        int top, int scoring, int n_groups, int keep, float scale) {
    extern __shared__ float route_smem[];                  // s [n_experts], c [n_experts], group scores [n_groups]
    float* s_of = route_smem;
    float* c_of = route_smem + n_experts;
    float* g_of = c_of + n_experts;
    pdl_trigger();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int token = blockIdx.x;
    if (positions != nullptr && positions[token] < 0) {
        for (int k = threadIdx.x; k < top; k += blockDim.x) {
            ids[(size_t)token * top + k] = -1;
            weights[(size_t)token * top + k] = 0.f;
        }
        if (gate != nullptr && threadIdx.x == 0) gate[token] = 0.f;
        return;
    }
    const T* row = h + (size_t)token * width;
    const bool vec = width % 4 == 0 && ((uintptr_t)w_router % 16 == 0) && (w_gate == nullptr || (uintptr_t)w_gate % 16 == 0);
    const int rows = n_experts + (gate != nullptr ? 1 : 0);
    for (int e = warp; e < rows; e += ROUTE_WARPS) {
        const float dot = route_dot(row, e < n_experts ? w_router + (size_t)e * width : w_gate, width, lane, vec);
        if (lane == 0) {
            if (e < n_experts) {
                const float s = scoring ? 1.0f / (1.0f + expf(-dot)) : dot;
                s_of[e] = s;
                c_of[e] = correction ? s + correction[e] : s;
            } else {
                gate[token] = 1.0f / (1.0f + expf(-dot));
            }
        }
    }
    __syncthreads();
    if (warp != 0) return;
    if (n_groups > 0) {
        const int per = n_experts / n_groups;
        for (int g = lane; g < n_groups; g += 32) {
            float a = -INFINITY, b = -INFINITY;            // the two largest of the group
            for (int e = g * per; e < (g + 1) * per; ++e) {
                const float v = c_of[e];
                if (v > a) b = a, a = v;
                else if (v > b) b = v;
            }
            g_of[g] = per > 1 ? a + b : a;
        }
        __syncwarp();
        // the `keep` best groups are marked by a score of +inf, then all others lose their experts
        for (int k = 0; k < keep; ++k) {
            float best = -INFINITY;
            int best_g = 0x7fffffff;
            for (int g = lane; g < n_groups; g += 32) {
                const float v = g_of[g];
                if (v != INFINITY && (v > best || (v == best && g < best_g))) best = v, best_g = g;
            }
            warp_argmax(best, best_g);
            if (best_g >= n_groups) {                      // scores that are not numbers: the first group not yet kept
                best_g = 0;
                while (best_g < n_groups - 1 && g_of[best_g] == INFINITY) ++best_g;
            }
            if (lane == 0) g_of[best_g] = INFINITY;
            __syncwarp();
        }
        for (int e = lane; e < n_experts; e += 32)
            if (g_of[e / per] != INFINITY) c_of[e] = -INFINITY;
        __syncwarp();
    }
    float first = 0.f, sum = 0.f;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int best_e = 0x7fffffff;
        for (int e = lane; e < n_experts; e += 32) {
            const float v = c_of[e];
            if (v > best || (v == best && e < best_e)) best = v, best_e = e;
        }
        warp_argmax(best, best_e);
        if (best_e >= n_experts) best_e = k;               // scores that are not numbers: still a valid choice
        const float s = s_of[best_e];
        float w = s * scale;
        if (!scoring) {
            if (k == 0) first = s;
            w = expf(s - first);
            sum += w;
        }
        if (lane == 0) {
            ids[(size_t)token * top + k] = best_e;
            weights[(size_t)token * top + k] = w;
            c_of[best_e] = -INFINITY;
        }
        __syncwarp();
    }
    if (!scoring) {
        const float inv = scale / sum;
        for (int k = lane; k < top; k += 32) weights[(size_t)token * top + k] *= inv;
    }
}

// ---- grouping -----------------------------------------------------------------------------------
// Block e finds the entries that chose expert e: offsets[e] = entries that chose a lower expert,
// and each of its entries gets slot offsets[e] + (its rank among them, in entry order).
constexpr int SORT_THREADS = 256;

__global__ void __launch_bounds__(SORT_THREADS)
moe_group_kernel(const int* __restrict__ ids, int n_entries, int n_experts, int* __restrict__ offsets,
                 int* __restrict__ slot_entry, int* __restrict__ entry_slot) {
    __shared__ int warp_count[SORT_THREADS / 32];
    __shared__ int total_less, total_equal, base;
    pdl_trigger();
    pdl_wait();
    const int e = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) total_less = 0, total_equal = 0, base = 0;
    __syncthreads();
    int less = 0, equal = 0;
    for (int i = tid; i < n_entries; i += SORT_THREADS) {
        const int id = ids[i];
        less += (id >= 0 && id < e);
        equal += (id == e);
    }
    less = __reduce_add_sync(0xffffffffu, less);
    equal = __reduce_add_sync(0xffffffffu, equal);
    if (lane == 0) atomicAdd(&total_less, less), atomicAdd(&total_equal, equal);
    __syncthreads();
    const int first = total_less;
    if (tid == 0) {
        offsets[e] = first;
        if (e == n_experts - 1) offsets[n_experts] = first + total_equal;
    }
    for (int i0 = 0; i0 < n_entries; i0 += SORT_THREADS) {
        const int i = i0 + tid;
        const int id = i < n_entries ? ids[i] : -1;
        const bool mine = id == e;
        const unsigned ballot = __ballot_sync(0xffffffffu, mine);
        if (lane == 0) warp_count[warp] = __popc(ballot);
        __syncthreads();
        int before = base;
        for (int w = 0; w < warp; ++w) before += warp_count[w];
        if (mine) {
            const int slot = first + before + __popc(ballot & ((1u << lane) - 1u));
            slot_entry[slot] = i;
            entry_slot[i] = slot;
        } else if (e == 0 && i < n_entries && (id < 0 || id >= n_experts)) {
            entry_slot[i] = -1;                            // an entry of a padding row
        }
        __syncthreads();
        if (tid == 0) {
            int add = 0;
            for (int w = 0; w < SORT_THREADS / 32; ++w) add += warp_count[w];
            base += add;
        }
        __syncthreads();
    }
}

// ---- the experts' matrix products over the groups ------------------------------------------------
// Tiles of 64 slots x 64 outputs, 16 of K at a time, on the CUDA cores (any sizes).  blockIdx.z is
// the expert, blockIdx.y the tile of its slots (tiles beyond its count leave at once).
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

__device__ __forceinline__ float silu(float z) { return z / (1.0f + expf(-z)); }

// The gated product of a unit's two hidden features g (gate) and u (up), by `act`:
//   0: silu(g) * u        1: g' * sigmoid(1.702 g') * (u' + 1), g' = min(g, limit), u' = clamp(u, -limit, limit)
//   2: gelu_tanh(g) * u
__device__ __forceinline__ float gated_value(int act, float limit, float g, float u) {
    if (act == 1) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
        return g / (1.0f + expf(-1.702f * g)) * (u + 1.0f);
    }
    if (act == 2) return gelu_tanh(g) * u;
    return silu(g) * u;
}

// GLU = true:  out[slot, n] = silu(a . w[e][n]) * (a . w[e][inner + n]),  a = x[token of slot]   (T out)
// GLU = false: out[slot, n] = scale[entry of slot] * (a . w[e][n]),       a = x[slot]            (32-bit out)
template <typename T, bool GLU>
__global__ void __launch_bounds__(256)
moe_gemm_kernel(const T* __restrict__ x, int ldx, const T* __restrict__ w, long long w_expert_stride,
                const int* __restrict__ offsets, const int* __restrict__ slot_entry, int top,
                const float* __restrict__ scale, void* __restrict__ out, int N, int K, int x_rows, int act, float limit) {
    __shared__ float as[BK][BM + 4];
    __shared__ float ws[BK][BN + 4];
    __shared__ float us[GLU ? BK : 1][BN + 4];
    __shared__ int row_of[BM];
    pdl_trigger();
    pdl_wait();
    const int e = blockIdx.z;
    const int first = offsets[e], count = offsets[e + 1] - first;
    const int m0 = blockIdx.y * BM;
    if (m0 >= count) return;
    const int n0 = blockIdx.x * BN;
    const int tid = threadIdx.x;
    if (tid < BM) {
        int r = -1;
        if (m0 + tid < count) {
            const int slot = first + m0 + tid;
            r = GLU ? slot_entry[slot] / top : slot;
            if (!MG_GUARDED(moe, MG_GUARD_ROW, r, x_rows)) r = -1;
        }
        row_of[tid] = r;
    }
    __syncthreads();
    const T* we = w + (size_t)e * w_expert_stride;
    const int tr = tid / 16, tc = tid % 16;
    float acc[TM][TN], acc_u[GLU ? TM : 1][GLU ? TN : 1];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            acc[i][j] = 0.f;
            if constexpr (GLU) acc_u[i][j] = 0.f;
        }
    const int lrow = tid >> 2, lk = (tid & 3) * 4;
    const int arow = row_of[lrow];
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int k = k0 + lk + i;
            const int n = n0 + lrow;
            as[lk + i][lrow] = (arow >= 0 && k < K) ? to_float(x[(size_t)arow * ldx + k]) : 0.f;
            ws[lk + i][lrow] = (n < N && k < K) ? to_float(we[(size_t)n * K + k]) : 0.f;
            if constexpr (GLU) us[lk + i][lrow] = (n < N && k < K) ? to_float(we[(size_t)(N + n) * K + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float av[TM], wv[TN], uv[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) av[i] = as[k][tr * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) {
                wv[j] = ws[k][tc * TN + j];
                if constexpr (GLU) uv[j] = us[k][tc * TN + j];
            }
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) {
                    acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
                    if constexpr (GLU) acc_u[i][j] = fmaf(av[i], uv[j], acc_u[i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + tr * TM + i;
        if (m >= count) continue;
        const size_t slot = (size_t)first + m;
        const float sc = GLU ? 1.f : scale[slot_entry[slot]];
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tc * TN + j;
            if (n >= N) continue;
            if constexpr (GLU)
                reinterpret_cast<T*>(out)[slot * N + n] = from_float<T>(gated_value(act, limit, acc[i][j], acc_u[i][j]));
            else
                reinterpret_cast<float*>(out)[slot * N + n] = acc[i][j] * sc;
        }
    }
}

// ---- the same products on the warp-level tensor cores (bfloat16, K a multiple of 8) -------------------
// Tiles of 64 slots x 128 rows of the expert's matrix, 64 of K at a time through two shared-memory
// buffers (cp.async: the next tile's copies are in flight while this one is multiplied); four warps as
// 2 x 2, each 32 slots x 64 matrix rows.  For the gated product a warp's 64 rows are 32 gate rows and
// the 32 up rows of the same outputs, so silu(gate) * up happens in the accumulators.
constexpr int MT = 64, MK = 64, MLD = MK + 8;
constexpr size_t moe_mma_smem(int mb, int stages) { return (size_t)stages * (MT + mb) * MLD * sizeof(bf16); }

__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix4(uint32_t (&r)[4], const bf16* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
// 16 bytes from global to shared memory, asynchronously; `real` false: zeros, nothing is read.
__device__ __forceinline__ void copy16_async(bf16* dst, const bf16* src, bool real) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    const int bytes = real ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}

// MB: rows of the expert's matrix per tile: 128 (four warps as 2 x 2, each 32 slots x 64 rows), or 64 for
// steps of few tokens (four warps as 4 x 1, each 16 slots x 64 rows): twice the CTAs, so that more of the
// matrices is in flight when the work is nothing but reading them.
// NS: shared-memory buffers that take turns (NS - 1 tiles are in flight while one is multiplied): two
// where many CTAs share an SM, four where a CTA does little but wait for its matrix.
template <bool GLU, int MB, int NS>
__global__ void __launch_bounds__(128)
moe_gemm_mma_kernel(const bf16* __restrict__ x, int ldx, const bf16* __restrict__ w, long long w_expert_stride,
                    const int* __restrict__ offsets, const int* __restrict__ slot_entry, int top,
                    const float* __restrict__ scale, void* __restrict__ out, int N, int K, int x_rows, int act, float limit) {
    extern __shared__ __align__(16) uint8_t moe_smem[];
    bf16* as = reinterpret_cast<bf16*>(moe_smem);          // [NS][MT * MLD]
    bf16* bs = as + NS * MT * MLD;                         // [NS][MB * MLD]
    __shared__ int row_of[MT];
    pdl_trigger();
    pdl_wait();
    const int e = blockIdx.z;
    const int first = offsets[e], count = offsets[e + 1] - first;
    const int m0 = blockIdx.y * MT;
    if (m0 >= count) return;
    const int n0 = blockIdx.x * (GLU ? MB / 2 : MB);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    constexpr int MI = MB == 128 ? 2 : 1;                  // m16 tiles per warp
    constexpr int BCH = MB * 8 / 128;                      // weight chunks per thread and tile
    if (tid < MT) {
        int r = -1;
        if (m0 + tid < count) {
            const int slot = first + m0 + tid;
            r = GLU ? slot_entry[slot] / top : slot;
            if (!MG_GUARDED(moe, MG_GUARD_ROW, r, x_rows)) r = -1;
        }
        row_of[tid] = r;
    }
    __syncthreads();
    const bf16* we = w + (size_t)e * w_expert_stride;
    // what this thread copies per tile: 4 chunks of 8 activations, 8 or 4 chunks of 8 weights
    const bf16* a_src[4];
    const bf16* b_src[BCH];
    const int chunk = (tid & 7) * 8;                       // the same column for all of a thread's chunks
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const int row = (tid + 128 * u) >> 3;
        a_src[u] = row_of[row] >= 0 ? x + (size_t)row_of[row] * ldx + chunk : nullptr;
    }
#pragma unroll
    for (int u = 0; u < BCH; ++u) {
        const int row = (tid + 128 * u) >> 3;
        int n, wrow;
        if (GLU) {
            const int r = row & 63;
            n = n0 + (row >> 6) * 32 + (r & 31);
            wrow = r < 32 ? n : N + n;
        } else {
            n = n0 + row;
            wrow = n;
        }
        b_src[u] = n < N ? we + (size_t)wrow * K + chunk : nullptr;
    }
    auto issue = [&](int buf, int k0) {
        const bool in_k = k0 + chunk < K;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const bool real = a_src[u] != nullptr && in_k;
            copy16_async(as + buf * MT * MLD + ((tid + 128 * u) >> 3) * MLD + chunk, real ? a_src[u] + k0 : x, real);
        }
#pragma unroll
        for (int u = 0; u < BCH; ++u) {
            const bool real = b_src[u] != nullptr && in_k;
            copy16_async(bs + buf * MB * MLD + ((tid + 128 * u) >> 3) * MLD + chunk, real ? b_src[u] + k0 : w, real);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    const int wr = MB == 128 ? warp >> 1 : warp, wc = MB == 128 ? warp & 1 : 0;
    const int m_warp = wr * 16 * MI;                       // the warp's first slot of the tile
    float acc[MI][8][4];
#pragma unroll
    for (int i = 0; i < MI; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f;
    const int iters = (K + MK - 1) / MK;
    // one group of copies per tile, also beyond the last tile (then empty), so that "all but the
    // newest NS - 1 groups have landed" always means: this iteration's tile is there
#pragma unroll
    for (int st = 0; st < NS - 1; ++st) {
        if (st < iters) issue(st, st * MK);
        else asm volatile("cp.async.commit_group;" ::: "memory");
    }
    for (int it = 0; it < iters; ++it) {
        const int buf = it % NS;
        if (it + NS - 1 < iters) issue((it + NS - 1) % NS, (it + NS - 1) * MK);
        else asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group %0;" ::"n"(NS - 1) : "memory");
        __syncthreads();
        const bf16* at = as + buf * MT * MLD;
        const bf16* bt = bs + buf * MB * MLD;
#pragma unroll
        for (int kk = 0; kk < MK / 16; ++kk) {
            uint32_t af[MI][4];
#pragma unroll
            for (int i = 0; i < MI; ++i)
                ldmatrix4(af[i], at + (m_warp + i * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * MLD + kk * 16 + (lane >> 4) * 8);
#pragma unroll
            for (int j = 0; j < 8; j += 2) {
                uint32_t bf[4];
                ldmatrix4(bf, bt + (wc * 64 + j * 8 + (lane >> 4) * 8 + (lane & 7)) * MLD + kk * 16 + ((lane >> 3) & 1) * 8);
#pragma unroll
                for (int i = 0; i < MI; ++i) {
                    mma_16816(acc[i][j], af[i], bf[0], bf[1]);
                    mma_16816(acc[i][j + 1], af[i], bf[2], bf[3]);
                }
            }
        }
        __syncthreads();                                    // the buffer is free for a later tile
    }
#pragma unroll
    for (int i = 0; i < MI; ++i)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int m = m0 + m_warp + i * 16 + (lane >> 2) + 8 * half;
            if (m >= count) continue;
            const size_t slot = (size_t)first + m;
            if (GLU) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int n = n0 + wc * 32 + j * 8 + 2 * (lane & 3);
                    const float v0 = gated_value(act, limit, acc[i][j][2 * half], acc[i][j + 4][2 * half]);
                    const float v1 = gated_value(act, limit, acc[i][j][2 * half + 1], acc[i][j + 4][2 * half + 1]);
                    bf16* o = reinterpret_cast<bf16*>(out) + slot * N + n;
                    if (n + 1 < N && (N & 1) == 0) *reinterpret_cast<__nv_bfloat162*>(o) = __floats2bfloat162_rn(v0, v1);
                    else {
                        if (n < N) o[0] = __float2bfloat16_rn(v0);
                        if (n + 1 < N) o[1] = __float2bfloat16_rn(v1);
                    }
                }
            } else {
                const float sc = scale[slot_entry[slot]];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int n = n0 + wc * 64 + j * 8 + 2 * (lane & 3);
                    float* o = reinterpret_cast<float*>(out) + slot * N + n;
                    if (n < N) o[0] = acc[i][j][2 * half] * sc;
                    if (n + 1 < N) o[1] = acc[i][j][2 * half + 1] * sc;
                }
            }
        }
}

// ---- x[token] += sum over the token's entries, in entry order ----------------------------------
__global__ void moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ entry_slot, int top,
                                   float* __restrict__ residual, int width, int n_slots) {
    pdl_trigger();
    pdl_wait();
    const int token = blockIdx.x;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float sum = 0.f;
        for (int k = 0; k < top; ++k) {
            const int slot = entry_slot[(size_t)token * top + k];
            if (slot >= 0 && MG_GUARDED(moe, MG_GUARD_ROW, slot, n_slots)) sum += y[(size_t)slot * width + c];
        }
        residual[(size_t)token * width + c] += sum;
    }
}

// ---- out[n, j] = silu(gu[n, j]) * gu[n, inner + j] (* scale[n]) -----------------------------------
template <typename T>
__global__ void glu_kernel(const T* __restrict__ gu, const float* __restrict__ scale, T* __restrict__ out, int rows,
                           int inner, int act, float limit) {
    pdl_trigger();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)rows * inner) return;
    const int n = (int)(i / inner), j = (int)(i - (long long)n * inner);
    const float g = to_float(gu[(size_t)n * 2 * inner + j]), u = to_float(gu[(size_t)n * 2 * inner + inner + j]);
    float v = gated_value(act, limit, g, u);
    if (scale != nullptr) v *= scale[n];
    out[i] = from_float<T>(v);
}

#define MG_LAUNCHED(e, name)                                                                 \
    do {                                                                                     \
        if ((e) != cudaSuccess) return mg_set_error(MG_ERR_CUDA, name ": %s", cudaGetErrorString(e)); \
    } while (0)

}  // namespace

// h: [n_tokens, width] (bfloat16 if is_bf16 else 32-bit); w_router: [n_experts, width] and w_gate:
// [width] (null: no gate), 32-bit; positions: [n_tokens] or null; ids, weights: [n_tokens, top];
// gate: [n_tokens] or null.
MG_API int mg_moe_route(const void* h, const float* w_router, const float* w_gate, const int* positions, int* ids,
                        float* weights, float* gate, int n_tokens, int width, int n_experts, int top, int is_bf16,
                        void* stream) {
    if (n_tokens == 0) return MG_OK;
    MG_REQUIRE(n_tokens > 0 && width > 0 && n_experts > 0 && top > 0 && top <= n_experts, "moe route: bad sizes");
    MG_REQUIRE((w_gate == nullptr) == (gate == nullptr), "moe route: a gate wants its weights and its output");
    const size_t smem = (size_t)n_experts * sizeof(float);
    MG_REQUIRE(smem <= 48 * 1024, "moe route: too many experts (%d)", n_experts);
    const dim3 grid(n_tokens), block(32 * ROUTE_WARPS);
    cudaError_t e;
    if (is_bf16)
        e = mg_launch(moe_route_kernel<bf16>, grid, block, smem, (cudaStream_t)stream, true, (const bf16*)h, w_router,
                      w_gate, positions, ids, weights, gate, n_tokens, width, n_experts, top);
    else
        e = mg_launch(moe_route_kernel<float>, grid, block, smem, (cudaStream_t)stream, true, (const float*)h, w_router,
                      w_gate, positions, ids, weights, gate, n_tokens, width, n_experts, top);
    MG_LAUNCHED(e, "moe route");
    return MG_OK;
}

// As mg_moe_route, with scores per expert (scoring 1: sigmoid, 0: the logits with a softmax over the chosen),
// correction: [n_experts] 32-bit or null, n_groups / keep: the groups (0: none), scale: factor on the weights.
MG_API int mg_moe_route_scored(const void* h, const float* w_router, const float* w_gate, const float* correction,
                               const int* positions, int* ids, float* weights, float* gate, int n_tokens, int width,
                               int n_experts, int top, int scoring, int n_groups, int keep, float scale, int is_bf16,
                               void* stream) {
    if (n_tokens == 0) return MG_OK;
    MG_REQUIRE(n_tokens > 0 && width > 0 && n_experts > 0 && top > 0 && top <= n_experts, "moe route: bad sizes");
    MG_REQUIRE((w_gate == nullptr) == (gate == nullptr), "moe route: a gate wants its weights and its output");
    MG_REQUIRE(n_groups >= 0 && (n_groups == 0 || (n_experts % n_groups == 0 && keep > 0 && keep <= n_groups &&
                                                   keep * (n_experts / n_groups) >= top)),
               "moe route: %d groups of which %d are kept do not fit %d experts and %d choices", n_groups, keep, n_experts, top);
    const size_t smem = (size_t)(2 * n_experts + n_groups) * sizeof(float);
    MG_REQUIRE(smem <= 48 * 1024, "moe route: too many experts (%d)", n_experts);
    const dim3 grid(n_tokens), block(32 * ROUTE_WARPS);
    cudaError_t e;
    if (is_bf16)
        e = mg_launch(moe_route_scored_kernel<bf16>, grid, block, smem, (cudaStream_t)stream, true, (const bf16*)h, w_router,
                      w_gate, correction, positions, ids, weights, gate, n_tokens, width, n_experts, top, scoring, n_groups,
                      keep, scale);
    else
        e = mg_launch(moe_route_scored_kernel<float>, grid, block, smem, (cudaStream_t)stream, true, (const float*)h, w_router,
                      w_gate, correction, positions, ids, weights, gate, n_tokens, width, n_experts, top, scoring, n_groups,
                      keep, scale);
    MG_LAUNCHED(e, "moe route (scored)");
    return MG_OK;
}

// ids: [n_entries] chosen experts (-1: none); offsets: [n_experts + 1]; slot_entry, entry_slot: [n_entries].
MG_API int mg_moe_group(const int* ids, int n_entries, int n_experts, int* offsets, int* slot_entry, int* entry_slot,
                        void* stream) {
    if (n_entries == 0) return MG_OK;
    MG_REQUIRE(n_entries > 0 && n_entries < (1 << 24) && n_experts > 0, "moe group: bad sizes");
    const cudaError_t e = mg_launch(moe_group_kernel, dim3(n_experts), dim3(SORT_THREADS), 0, (cudaStream_t)stream, true,
                                    ids, n_entries, n_experts, offsets, slot_entry, entry_slot);
    MG_LAUNCHED(e, "moe group");
    return MG_OK;
}

// act, limit: the gated product of the first product's two halves (see gated_value).
// glu = 1: x [x_rows, ldx] gathered by token, w [n_experts, 2 N, K], out [n_entries, N] in the inputs' type.
// glu = 0: x [n_entries, ldx] by slot, w [n_experts, N, K], scale [n_entries] by entry, out [n_entries, N] 32-bit.
// max_rows: the most slots one expert can have (the tokens of the step).
MG_API int mg_moe_gemm(const void* x, int ldx, const void* w, const int* offsets, const int* slot_entry, int top,
                       const float* scale, void* out, int n_experts, int max_rows, int N, int K, int x_rows, int glu,
                       int is_bf16, int act, float limit, void* stream) {
    if (max_rows == 0) return MG_OK;
    MG_REQUIRE(n_experts > 0 && n_experts <= 65535 && max_rows > 0 && N > 0 && K > 0 && ldx >= K && top > 0,
               "moe gemm: bad sizes");
    MG_REQUIRE(glu || scale != nullptr, "moe gemm: the second product wants the entries' weights");
    const dim3 grid(ceil_div(N, BN), ceil_div(max_rows, BM), n_experts), block(256);
    MG_REQUIRE(grid.y <= 65535, "moe gemm: too many rows");
    const long long stride = (long long)(glu ? 2 : 1) * N * K;
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e;
    const bool tensor_cores = is_bf16 && K % 8 == 0 && ldx % 8 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)w % 16 == 0 &&
                              (uintptr_t)out % 4 == 0;
    if (tensor_cores) {
        const bool few = max_rows <= MT;                    // few tokens: narrower tiles, more CTAs
        const int mb = few ? 64 : 128;
        const dim3 tgrid(ceil_div(N, glu ? mb / 2 : mb), ceil_div(max_rows, MT), n_experts);
        static bool configured = false;
        if (!configured) {
            e = cudaFuncSetAttribute(moe_gemm_mma_kernel<true, 128, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)moe_mma_smem(128, 2));
            if (e == cudaSuccess)
                e = cudaFuncSetAttribute(moe_gemm_mma_kernel<false, 128, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)moe_mma_smem(128, 2));
            if (e == cudaSuccess)
                e = cudaFuncSetAttribute(moe_gemm_mma_kernel<true, 64, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)moe_mma_smem(64, 4));
            if (e == cudaSuccess)
                e = cudaFuncSetAttribute(moe_gemm_mma_kernel<false, 64, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)moe_mma_smem(64, 4));
            MG_LAUNCHED(e, "moe gemm (shared memory)");
            configured = true;
        }
        const bf16* xb = (const bf16*)x;
        const bf16* wb = (const bf16*)w;
        if (glu && few)
            e = mg_launch(moe_gemm_mma_kernel<true, 64, 4>, tgrid, dim3(128), moe_mma_smem(64, 4), s, true, xb, ldx, wb, stride,
                          offsets, slot_entry, top, scale, out, N, K, x_rows, act, limit);
        else if (glu)
            e = mg_launch(moe_gemm_mma_kernel<true, 128, 2>, tgrid, dim3(128), moe_mma_smem(128, 2), s, true, xb, ldx, wb, stride,
                          offsets, slot_entry, top, scale, out, N, K, x_rows, act, limit);
        else if (few)
            e = mg_launch(moe_gemm_mma_kernel<false, 64, 4>, tgrid, dim3(128), moe_mma_smem(64, 4), s, true, xb, ldx, wb, stride,
                          offsets, slot_entry, top, scale, out, N, K, x_rows, act, limit);
        else
            e = mg_launch(moe_gemm_mma_kernel<false, 128, 2>, tgrid, dim3(128), moe_mma_smem(128, 2), s, true, xb, ldx, wb, stride,
                          offsets, slot_entry, top, scale, out, N, K, x_rows, act, limit);
    } else if (is_bf16 && glu)
        e = mg_launch(moe_gemm_kernel<bf16, true>, grid, block, 0, s, true, (const bf16*)x, ldx, (const bf16*)w, stride,
                      offsets, slot_entry, top, scale, out, N, K, x_rows, act, limit);
    else if (is_bf16)
        e = mg_launch(moe_gemm_kernel<bf16, false>, grid, block, 0, s, true, (const bf16*)x, ldx, (const bf16*)w, stride,
                      offsets, slot_entry, top, scale, out, N, K, x_rows, act, limit);
    else if (glu)
        e = mg_launch(moe_gemm_kernel<float, true>, grid, block, 0, s, true, (const float*)x, ldx, (const float*)w, stride,
                      offsets, slot_entry, top, scale, out, N, K, x_rows, act, limit);
    else
        e = mg_launch(moe_gemm_kernel<float, false>, grid, block, 0, s, true, (const float*)x, ldx, (const float*)w,
                      stride, offsets, slot_entry, top, scale, out, N, K, x_rows, act, limit);
    MG_LAUNCHED(e, "moe gemm");
    return MG_OK;
}

// y: [n_slots, width] 32-bit; entry_slot: [n_tokens, top] (-1: none); residual: [n_tokens, width] 32-bit.
MG_API int mg_moe_combine(const float* y, const int* entry_slot, int top, float* residual, int n_tokens, int width,
                          int n_slots, void* stream) {
    if (n_tokens == 0) return MG_OK;
    MG_REQUIRE(n_tokens > 0 && width > 0 && top > 0, "moe combine: bad sizes");
    const cudaError_t e = mg_launch(moe_combine_kernel, dim3(n_tokens), dim3(width >= 256 ? 256 : 128), 0,
                                    (cudaStream_t)stream, true, y, entry_slot, top, residual, width, n_slots);
    MG_LAUNCHED(e, "moe combine");
    return MG_OK;
}

// gu: [rows, 2 inner] (gate columns first); scale: [rows] 32-bit or null; out: [rows, inner].
MG_API int mg_glu(const void* gu, const float* scale, void* out, int rows, int inner, int is_bf16, int act, float limit,
                  void* stream) {
    if (rows == 0) return MG_OK;
    MG_REQUIRE(rows > 0 && inner > 0, "glu: bad sizes");
    const long long n = (long long)rows * inner;
    const dim3 grid((unsigned)((n + 255) / 256)), block(256);
    cudaError_t e;
    if (is_bf16)
        e = mg_launch(glu_kernel<bf16>, grid, block, 0, (cudaStream_t)stream, true, (const bf16*)gu, scale, (bf16*)out,
                      rows, inner, act, limit);
    else
        e = mg_launch(glu_kernel<float>, grid, block, 0, (cudaStream_t)stream, true, (const float*)gu, scale, (float*)out,
                      rows, inner, act, limit);
    MG_LAUNCHED(e, "glu");
    return MG_OK;
}
