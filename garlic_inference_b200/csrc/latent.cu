// Latent attention, the step between the projections and the attention kernel: the new token's latent row
// goes into the paged cache and the queries are put into the form the attention kernel reads.
//
// A token's cache row is [ c (kv_rank) | rotated shared key part (rot_dim) | zeros up to the row's width ],
// c = rmsnorm(first kv_rank columns of the down-projection) * w.  Every head's key is W_uk,h c beside the
// shared rotated part and its value is W_uv,h c, so with q'_h = W_uk,h^T q_h (made by a per-head product
// before this kernel) the score is  q'_h . c + rot(q_rot,h) . rot(k_rot),  attention over the cache rows
// themselves gives sum_j p_j c_j, and W_uv,h is applied to that afterwards: the cache is read once for all
// heads and keys and values are never expanded.
//
// Rotation: pair (2i, 2i+1) of the rotated part, i < n_rot / 2, turns by the float32 product
// position * freq[i]; cosine and sine are multiplied by `magnitude`; dimensions from n_rot on pass.
// NikolayBlagoev/garlic-inference has one attention (grouped-query, src/models/qwen3/qwen3.cpp:140-179) and
// the rotate-half layout (src/src-cuda/rope.cu:41-79).
#include "common.cuh"
#include <math.h>

template <typename T>
__global__ void latent_prepare_kernel(const T* __restrict__ proj, long long ld, int q_off, int c_off,
                                      const T* __restrict__ q_lat, const void* __restrict__ norm_w, int w_dtype,
                                      float eps, const float* __restrict__ freq, float magnitude, int n_rot,
                                      const int* __restrict__ tok_pos, const int* __restrict__ tok_slot,
                                      const int* __restrict__ block_table, T* __restrict__ pool,
                                      T* __restrict__ q_out, int H, int d, int dr, int rank, int row_w,
                                      int page_size, int max_pages, int n_pool_pages, int append,
                                      int* __restrict__ status) {
    gi_pdl_start();
    __shared__ float red[33];
    const int t = blockIdx.x;
    const int pos = tok_pos[t], slot = tok_slot[t];
    const T* row = proj + (size_t)t * ld;
    const float p = (float)pos;

    // queries: [ q' (rank) | rotated part (dr) | zeros ] per head
    for (int i = threadIdx.x; i < H * row_w; i += blockDim.x) {
        const int h = i / row_w, c = i - h * row_w;
        float v = 0.f;
        if (c < rank) {
            v = to_f32(q_lat[((size_t)t * H + h) * rank + c]);
        } else if (c < rank + dr) {
            const int j = c - rank;
            const T* qr = row + q_off + (size_t)h * (d + dr) + d;
            if (j < n_rot) {
                float sn, cs;
                sincosf(p * freq[j >> 1], &sn, &cs);
                sn *= magnitude; cs *= magnitude;
                const float a = to_f32(qr[j & ~1]), b = to_f32(qr[j | 1]);
                v = (j & 1) ? b * cs + a * sn : a * cs - b * sn;
            } else {
                v = to_f32(qr[j]);
            }
        }
        q_out[((size_t)t * H + h) * row_w + c] = from_f32<T>(v);
    }
    if (!append || slot < 0) return;
    const int lp = pos / page_size;
    if (pos < 0 || lp >= max_pages) { if (threadIdx.x == 0) atomicExch(status, 1); return; }
    const int page = block_table[(size_t)slot * max_pages + lp];
    if (page < 0 || page >= n_pool_pages) { if (threadIdx.x == 0) atomicExch(status, 2); return; }
    T* dst = pool + ((size_t)page * page_size + (pos - lp * page_size)) * row_w;

    const T* cr = row + c_off;
    float ss = 0.f;
    for (int c = threadIdx.x; c < rank; c += blockDim.x) { const float x = to_f32(cr[c]); ss += x * x; }
    ss = block_sum(ss, red);
    const float inv = 1.f / sqrtf(ss / (float)rank + eps);
    for (int c = threadIdx.x; c < row_w; c += blockDim.x) {
        float v = 0.f;
        if (c < rank) {
            v = to_f32(cr[c]) * inv * load_w(norm_w, w_dtype, c);
        } else if (c < rank + dr) {
            const int j = c - rank;
            const T* kr = cr + rank;
            if (j < n_rot) {
                float sn, cs;
                sincosf(p * freq[j >> 1], &sn, &cs);
                sn *= magnitude; cs *= magnitude;
                const float a = to_f32(kr[j & ~1]), b = to_f32(kr[j | 1]);
                v = (j & 1) ? b * cs + a * sn : a * cs - b * sn;
            } else {
                v = to_f32(kr[j]);
            }
        }
        dst[c] = from_f32<T>(v);
    }
}

extern "C" int gi_latent_prepare(const void* proj, long long ld, int q_off, int c_off, const void* q_lat,
                                 int act_dtype, const void* norm_w, int w_dtype, float eps, const float* freq,
                                 float magnitude, int n_rot, const int* tok_pos, const int* tok_slot,
                                 const int* block_table, void* pool, void* q_out, int n_tokens, int H, int d, int dr,
                                 int rank, int row_w, int page_size, int max_pages, int n_pool_pages, int append,
                                 int* status, void* stream) {
    GI_REQUIRE(n_tokens >= 0 && H > 0 && d > 0 && dr >= 0 && rank > 0, "gi_latent_prepare: sizes must be positive");
    GI_REQUIRE(row_w >= rank + dr, "gi_latent_prepare: cache rows of %d hold no latent of %d and key part of %d",
               row_w, rank, dr);
    GI_REQUIRE(n_rot % 2 == 0 && n_rot <= dr, "gi_latent_prepare: %d rotated dimensions of %d", n_rot, dr);
    if (n_tokens == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (act_dtype == GI_DTYPE_F32)
        gi_launch(latent_prepare_kernel<float>, dim3(n_tokens), dim3(128), 0, s, (const float*)proj, ld, q_off, c_off,
                  (const float*)q_lat, norm_w, w_dtype, eps, freq, magnitude, n_rot, tok_pos, tok_slot, block_table,
                  (float*)pool, (float*)q_out, H, d, dr, rank, row_w, page_size, max_pages, n_pool_pages, append, status);
    else if (act_dtype == GI_DTYPE_BF16)
        gi_launch(latent_prepare_kernel<bf16>, dim3(n_tokens), dim3(128), 0, s, (const bf16*)proj, ld, q_off, c_off,
                  (const bf16*)q_lat, norm_w, w_dtype, eps, freq, magnitude, n_rot, tok_pos, tok_slot, block_table,
                  (bf16*)pool, (bf16*)q_out, H, d, dr, rank, row_w, page_size, max_pages, n_pool_pages, append, status);
    else
        GI_REQUIRE(false, "gi_latent_prepare: activation dtype %d", act_dtype);
    return gi_check_launch("gi_latent_prepare");
}
