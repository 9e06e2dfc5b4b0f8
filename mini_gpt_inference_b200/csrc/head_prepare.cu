// What happens to a fused projection's query, key and value heads between the projection and the
// attention, as one kernel: unit-RMS normalisation of query and key heads, the blend of the values
// with another layer's values of the same token, and the write of keys and values to their pages.
//
// One warp per (token, head) over the H query heads, the G key heads and the G value heads of a row
// [ ... q (H x D) ... k (G x D) ... v (G x Dv) ... ] whose three column offsets are parameters.
//   query head:  q <- q / sqrt(mean(q^2) + eps), in place            (if unit_norm)
//   key head:    k <- k / sqrt(mean(k^2) + eps), to its cache row    (if unit_norm; else copied)
//   value head:  v <- (1 - t) v + t v_other,      to its cache row    (if v_other is given; else copied)
// With q_gain / k_gain (head_dim numbers each, shared by the heads) the unit-RMS query and key heads
// are multiplied by them.  The value columns may be the key columns (v_off = k_off): keys are
// normalised on their way to the cache, never in place, so the values are the keys as projected.
// The statistics and the blend are 32-bit; t is read from device memory.  Key pages are
// [page, kv head, page_tokens, D], value pages [page, kv head, page_tokens, Dv].  A token with a
// negative position (padding of a fixed-size batch) is skipped, a negative cache row is not written.
#include "common.cuh"

MG_GUARD_DECLARE(head_prepare)

namespace {

constexpr int WARPS = 4;
constexpr int MAX_PER_LANE = 8;     // head sizes up to 256

template <typename T>
__global__ void __launch_bounds__(32 * WARPS)
head_prepare_kernel(T* __restrict__ proj, int ld, int n_tokens, int n_head, int n_kv_head, int head_dim, int v_dim,
                    int q_off, int k_off, int v_off, int unit_norm, float eps, const T* __restrict__ v_other,
                    int v_other_ld, const float* __restrict__ blend, const int* __restrict__ slots,
                    const int* __restrict__ positions, T* __restrict__ k_pages, T* __restrict__ v_pages,
                    int page_tokens, int num_pages, const float* __restrict__ q_gain, const float* __restrict__ k_gain) {
    pdl_trigger();
    pdl_wait();                                            // the rows come from the projection in front
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int token = blockIdx.x;
    const int unit = blockIdx.y * WARPS + warp;
    if (unit >= n_head + 2 * n_kv_head) return;
    if (positions != nullptr && positions[token] < 0) return;
    T* row = proj + (size_t)token * ld;
    int slot = slots ? slots[token] : -1;
    if (slot >= 0 && !MG_GUARDED(head_prepare, MG_GUARD_CACHE_ROW, slot, (long long)num_pages * page_tokens)) slot = -1;
    const int page = slot >= 0 ? slot / page_tokens : 0, within = slot >= 0 ? slot - page * page_tokens : 0;

    if (unit < n_head + n_kv_head) {                       // a query or key head
        const bool is_key = unit >= n_head;
        const int h = is_key ? unit - n_head : unit;
        T* src = row + (is_key ? k_off : q_off) + (size_t)h * head_dim;
        float v[MAX_PER_LANE];
        float sq = 0.f;
#pragma unroll
        for (int i = 0; i < MAX_PER_LANE; ++i) {
            const int d = lane + 32 * i;
            v[i] = d < head_dim ? to_float(src[d]) : 0.f;
            sq = fmaf(v[i], v[i], sq);
        }
        const float r = unit_norm ? 1.0f / sqrtf(warp_sum(sq) / (float)head_dim + eps) : 1.0f;
        const float* gain = is_key ? k_gain : q_gain;
        T* dst = src;
        if (is_key) {
            if (k_pages == nullptr || slot < 0) return;
            dst = k_pages + (((size_t)page * n_kv_head + h) * page_tokens + within) * head_dim;
        } else if (!unit_norm) {
            return;
        }
#pragma unroll
        for (int i = 0; i < MAX_PER_LANE; ++i) {
            const int d = lane + 32 * i;
            if (d < head_dim) dst[d] = from_float<T>(gain ? v[i] * r * gain[d] : v[i] * r);
        }
        return;
    }
    // a value head
    if (v_pages == nullptr || slot < 0) return;
    const int h = unit - n_head - n_kv_head;
    const T* src = row + v_off + (size_t)h * v_dim;
    const T* other = v_other ? v_other + (size_t)token * v_other_ld + (size_t)h * v_dim : nullptr;
    const float t = other ? blend[0] : 0.f;
    T* dst = v_pages + (((size_t)page * n_kv_head + h) * page_tokens + within) * v_dim;
    for (int d = lane; d < v_dim; d += 32) {
        float x = to_float(src[d]);
        if (other) x = (1.0f - t) * x + t * to_float(other[d]);
        dst[d] = from_float<T>(x);
    }
}

}  // namespace

// proj: [n_tokens, ld] rows of a fused projection (bfloat16 if is_bf16 else 32-bit), modified in place
// (query heads); v_other: [n_tokens, v_other_ld] rows whose first n_kv_head * v_dim columns are the
// values to blend in, blend: one 32-bit number on the device (both null: no blend); slots: [n_tokens]
// flat cache rows (null with the pages: nothing is cached); positions: [n_tokens] or null; q_gain, k_gain:
// [head_dim] 32-bit or null.
MG_API int mg_head_prepare(void* proj, int ld, int n_tokens, int n_head, int n_kv_head, int head_dim, int v_dim,
                           int q_off, int k_off, int v_off, int unit_norm, float eps, const void* v_other,
                           int v_other_ld, const float* blend, const int* slots, const int* positions, void* k_pages,
                           void* v_pages, int page_tokens, int num_pages, int is_bf16, const float* q_gain,
                           const float* k_gain, void* stream) {
    if (n_tokens == 0) return MG_OK;
    MG_REQUIRE(n_tokens > 0 && n_head > 0 && n_kv_head > 0 && head_dim > 0 && v_dim > 0, "head_prepare: bad sizes");
    MG_REQUIRE(head_dim <= 32 * MAX_PER_LANE && v_dim <= 32 * MAX_PER_LANE, "head_prepare: heads of up to %d features",
               32 * MAX_PER_LANE);
    MG_REQUIRE(q_off >= 0 && k_off >= 0 && v_off >= 0 && q_off + n_head * head_dim <= ld &&
                   k_off + n_kv_head * head_dim <= ld && v_off + n_kv_head * v_dim <= ld,
               "head_prepare: heads outside the rows");
    MG_REQUIRE((q_gain == nullptr && k_gain == nullptr) || unit_norm, "head_prepare: gains without the unit norm");
    MG_REQUIRE((v_other == nullptr) == (blend == nullptr), "head_prepare: a blend wants both the other values and its weight");
    MG_REQUIRE(v_other == nullptr || v_other_ld >= n_kv_head * v_dim, "head_prepare: the other values' rows are too short");
    MG_REQUIRE((k_pages == nullptr) == (v_pages == nullptr) && (k_pages == nullptr || (slots && page_tokens > 0)),
               "head_prepare: pages without cache rows");
    const dim3 grid(n_tokens, ceil_div(n_head + 2 * n_kv_head, WARPS)), block(32 * WARPS);
    MG_REQUIRE(grid.y <= 65535, "head_prepare: too many heads");
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e;
    if (is_bf16)
        e = mg_launch(head_prepare_kernel<bf16>, grid, block, 0, s, true, (bf16*)proj, ld, n_tokens, n_head, n_kv_head,
                      head_dim, v_dim, q_off, k_off, v_off, unit_norm, eps, (const bf16*)v_other, v_other_ld, blend, slots,
                      positions, (bf16*)k_pages, (bf16*)v_pages, page_tokens, num_pages, q_gain, k_gain);
    else
        e = mg_launch(head_prepare_kernel<float>, grid, block, 0, s, true, (float*)proj, ld, n_tokens, n_head, n_kv_head,
                      head_dim, v_dim, q_off, k_off, v_off, unit_norm, eps, (const float*)v_other, v_other_ld, blend, slots,
                      positions, (float*)k_pages, (float*)v_pages, page_tokens, num_pages, q_gain, k_gain);
    if (e != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "head_prepare: %s", cudaGetErrorString(e));
    return MG_OK;
}
