// Causal softmax over rows of scores that a matrix product left in float32, with an optional sink, for
// attention done as product - softmax - product (prompts of mixers whose keys and values are shared by all heads,
// where both products are plain matrix products over [tokens x heads] rows).
//
// Row r = t * heads + h holds the scores of query token t (position first_pos + t) and head h against keys
// 0 .. n_keys-1 (columns).  Keys beyond the query's position get weight 0.  With m = max(max_j s_j scale, sink_h):
//   p_j = exp(s_j scale - m) / ( sum_j exp(s_j scale - m) + exp(sink_h - m) )
// The sink has no column: it only joins the denominator.  Scores, maximum, sum and weights are float32; the
// weights are rounded once to the type of the second product's operand.
// NikolayBlagoev/garlic-inference leaves softmax to its attention library (src/src-cuda/attention/fattn.cu:74-86).
#include "common.cuh"
#include <math.h>

template <typename T>
__global__ void causal_sink_softmax_kernel(const float* __restrict__ s, long long lds, T* __restrict__ p, long long ldp,
                                           int heads, int first_pos, int n_keys, float scale,
                                           const void* __restrict__ sinks, int sink_dtype) {
    gi_pdl_start();
    __shared__ float red[33];
    const size_t r = blockIdx.x;
    const int t = (int)(r / heads), h = (int)(r - (size_t)t * heads);
    const int last = min(first_pos + t, n_keys - 1);            // keys 0..last are seen
    const float* row = s + r * lds;
    T* out = p + r * ldp;
    float m = sinks ? load_w(sinks, sink_dtype, h) : -INFINITY;
    const float sink = m;
    for (int j = threadIdx.x; j <= last; j += blockDim.x) m = fmaxf(m, row[j] * scale);
    // block maximum: lane tree, then warps
    m = warp_max(m);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        float v = red[0];
        for (int w = 1; w < (int)((blockDim.x + 31) >> 5); ++w) v = fmaxf(v, red[w]);
        red[32] = v;
    }
    __syncthreads();
    m = red[32];
    float sum = 0.f;
    for (int j = threadIdx.x; j <= last; j += blockDim.x) sum += expf(row[j] * scale - m);
    sum = block_sum(sum, red);
    if (sinks) sum += expf(sink - m);
    const float inv = 1.f / sum;
    for (int j = threadIdx.x; j < n_keys; j += blockDim.x)
        out[j] = from_f32<T>(j <= last ? expf(row[j] * scale - m) * inv : 0.f);
}

extern "C" int gi_causal_sink_softmax(const float* s, long long lds, void* p, long long ldp, int p_dtype, int n_rows,
                                      int heads, int first_pos, int n_keys, float scale, const void* sinks,
                                      int sink_dtype, void* stream) {
    GI_REQUIRE(n_rows >= 0 && heads > 0 && n_keys > 0 && first_pos >= 0 && n_rows % heads == 0,
               "gi_causal_sink_softmax: %d rows of %d heads, %d keys", n_rows, heads, n_keys);
    GI_REQUIRE(lds >= n_keys && ldp >= n_keys, "gi_causal_sink_softmax: row strides shorter than the rows");
    if (n_rows == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    if (p_dtype == GI_DTYPE_F32)
        gi_launch(causal_sink_softmax_kernel<float>, dim3(n_rows), dim3(256), 0, st, s, lds, (float*)p, ldp, heads,
                  first_pos, n_keys, scale, sinks, sink_dtype);
    else if (p_dtype == GI_DTYPE_BF16)
        gi_launch(causal_sink_softmax_kernel<bf16>, dim3(n_rows), dim3(256), 0, st, s, lds, (bf16*)p, ldp, heads,
                  first_pos, n_keys, scale, sinks, sink_dtype);
    else
        GI_REQUIRE(false, "gi_causal_sink_softmax: output dtype %d", p_dtype);
    return gi_check_launch("gi_causal_sink_softmax");
}
