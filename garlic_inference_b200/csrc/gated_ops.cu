// Row-wise kernels of layers whose sublayer results are gated and normed before they join the residual
// stream, and of mixers whose read-out is normed per group and gated.
//
//   gi_gate_norm_add        x += rmsnorm( y * sigmoid(g + b) ) * w     (x the float32 residual stream; the gate is
//                           optional), with a copy of the new x in the activation type for the next products
//   gi_xielu                a(z) = softplus(p) z^2 + z/2                         z > 0
//                                  (1/2 + softplus(q)) (e^z - 1 - z) + z/2       z <= 0
//   gi_gated_group_rmsnorm  out = o / rms(o over its group) * w * gate(g),  gate = sigmoid or silu
//
// Everything is float32 inside and rounded once on the way out; T is the activation type.  Block sizes depend
// on the row's width alone, so a row's result does not depend on what else is in the launch.
// NikolayBlagoev/garlic-inference has none of these (its one layer is pre-norm with a plain residual add,
// src/src-cuda/norm.cu:51-101).
#include "common.cuh"
#include <math.h>

__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// ------------------------------------------------------------------ gate, norm, add
// Eight consecutive values starting at element c (a multiple of 8, the base on 16 bytes) as float32.
__device__ __forceinline__ void load8(const float* p, int c, float* out) {
    const float4 a = *reinterpret_cast<const float4*>(p + c), b = *reinterpret_cast<const float4*>(p + c + 4);
    out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w; out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
}
__device__ __forceinline__ void load8(const bf16* p, int c, float* out) {
    const uint4 w = *reinterpret_cast<const uint4*>(p + c);
    const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&w);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(p2[i]); out[2 * i] = f.x; out[2 * i + 1] = f.y; }
}
__device__ __forceinline__ void load8_w(const void* w, int w_dtype, int c, float* out) {
    if (w_dtype == GI_DTYPE_F32) load8((const float*)w, c, out); else load8((const bf16*)w, c, out);
}
__device__ __forceinline__ void store8(float* p, int c, const float* v) {
    *reinterpret_cast<float4*>(p + c) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + c + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void store8(bf16* p, int c, const float* v) {
    uint4 w;
    __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&w);
#pragma unroll
    for (int i = 0; i < 4; ++i) p2[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p + c) = w;
}

// The same arithmetic as the kernel below, element for element, with 16-byte loads and stores (a thread sums
// eight consecutive elements at a time, then the block's tree): taken when the rows allow it, which depends
// on the sizes and the tensors' alignment alone, never on how a request was cut.  A decode step runs this kernel twice per layer on a handful of rows, where it is a chain of
// memory latencies, so the fewer and wider its loads the better.
template <typename T>
__global__ void gate_norm_add_vec_kernel(const T* __restrict__ y, long long ldy, const T* __restrict__ g, long long ldg,
                                         const void* __restrict__ bias, int b_dtype, const void* __restrict__ weight,
                                         int w_dtype, float* __restrict__ residual, T* __restrict__ act_out, int dim,
                                         float eps) {
    gi_pdl_start();
    extern __shared__ float row[];
    float* red = row + dim;
    const size_t r = blockIdx.x;
    const T* yr = y + r * ldy;
    const T* gr = g ? g + r * ldg : nullptr;
    float ss = 0.f;
#pragma unroll 2
    for (int c = threadIdx.x * 8; c < dim; c += blockDim.x * 8) {
        float s[8], z[8], b[8];
        load8(yr, c, s);
        if (gr) {
            load8(gr, c, z);
            if (bias) load8_w(bias, b_dtype, c, b);
#pragma unroll
            for (int i = 0; i < 8; ++i) s[i] *= sigmoid_f(z[i] + (bias ? b[i] : 0.f));
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) { row[c + i] = s[i]; ss += s[i] * s[i]; }
    }
    ss = block_sum(ss, red);
    const float inv = 1.f / sqrtf(ss / (float)dim + eps);
    float* res = residual + r * dim;
#pragma unroll 2
    for (int c = threadIdx.x * 8; c < dim; c += blockDim.x * 8) {
        float x[8], w[8];
        load8(res, c, x);
        load8_w(weight, w_dtype, c, w);
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] += row[c + i] * inv * w[i];
        store8(res, c, x);
        if (act_out) store8(act_out + r * dim, c, x);
    }
}

template <typename T>
__global__ void gate_norm_add_kernel(const T* __restrict__ y, long long ldy, const T* __restrict__ g, long long ldg,
                                     const void* __restrict__ bias, int b_dtype, const void* __restrict__ weight,
                                     int w_dtype, float* __restrict__ residual, T* __restrict__ act_out, int dim,
                                     float eps) {
    gi_pdl_start();
    extern __shared__ float row[];               // dim gated values, then 33 for the reduction
    float* red = row + dim;
    const size_t r = blockIdx.x;
    const T* yr = y + r * ldy;
    const T* gr = g ? g + r * ldg : nullptr;
    float ss = 0.f;
    // unrolled: a few rows at a time are one chain of memory latencies, so the loads of several iterations go out together
#pragma unroll 8
    for (int c = threadIdx.x; c < dim; c += blockDim.x) {
        float s = to_f32(yr[c]);
        if (gr) s *= sigmoid_f(to_f32(gr[c]) + (bias ? load_w(bias, b_dtype, c) : 0.f));
        row[c] = s;
        ss += s * s;
    }
    ss = block_sum(ss, red);
    const float inv = 1.f / sqrtf(ss / (float)dim + eps);
    float* res = residual + r * dim;
#pragma unroll 8
    for (int c = threadIdx.x; c < dim; c += blockDim.x) {
        const float x = res[c] + row[c] * inv * load_w(weight, w_dtype, c);
        res[c] = x;
        if (act_out) act_out[r * dim + c] = from_f32<T>(x);
    }
}

extern "C" int gi_gate_norm_add(const void* y, long long ldy, const void* g, long long ldg, const void* bias,
                                int b_dtype, const void* weight, int w_dtype, float* residual, void* act_out,
                                int act_dtype, int n_rows, int dim, float eps, void* stream) {
    GI_REQUIRE(n_rows >= 0 && dim > 0 && dim <= 16384, "gi_gate_norm_add: rows of %d elements (at most 16384)", dim);
    GI_REQUIRE(ldy >= dim && (!g || ldg >= dim), "gi_gate_norm_add: row strides shorter than the rows");
    if (n_rows == 0) return 0;
    const int threads = dim >= 4096 ? 512 : (dim >= 1024 ? 256 : 128);
    const size_t smem = ((size_t)dim + 33) * sizeof(float);
    cudaStream_t s = (cudaStream_t)stream;
    auto on16 = [](const void* p) { return p == nullptr || (uintptr_t)p % 16 == 0; };
    const bool vec = dim % 8 == 0 && ldy % 8 == 0 && (!g || ldg % 8 == 0) && on16(y) && on16(g) && on16(bias) &&
                     on16(weight) && on16(residual) && on16(act_out) && smem <= 48 * 1024;
    if (vec && act_dtype == GI_DTYPE_F32) {
        gi_launch(gate_norm_add_vec_kernel<float>, dim3(n_rows), dim3(threads), smem, s, (const float*)y, ldy, (const float*)g,
                  ldg, bias, b_dtype, weight, w_dtype, residual, (float*)act_out, dim, eps);
    } else if (vec && act_dtype == GI_DTYPE_BF16) {
        gi_launch(gate_norm_add_vec_kernel<bf16>, dim3(n_rows), dim3(threads), smem, s, (const bf16*)y, ldy, (const bf16*)g,
                  ldg, bias, b_dtype, weight, w_dtype, residual, (bf16*)act_out, dim, eps);
    } else if (act_dtype == GI_DTYPE_F32) {
        if (smem > 48 * 1024) { int rc = gi_reserve_smem((const void*)gate_norm_add_kernel<float>, smem, "gi_gate_norm_add"); if (rc) return rc; }
        gi_launch(gate_norm_add_kernel<float>, dim3(n_rows), dim3(threads), smem, s, (const float*)y, ldy, (const float*)g,
                  ldg, bias, b_dtype, weight, w_dtype, residual, (float*)act_out, dim, eps);
    } else if (act_dtype == GI_DTYPE_BF16) {
        if (smem > 48 * 1024) { int rc = gi_reserve_smem((const void*)gate_norm_add_kernel<bf16>, smem, "gi_gate_norm_add"); if (rc) return rc; }
        gi_launch(gate_norm_add_kernel<bf16>, dim3(n_rows), dim3(threads), smem, s, (const bf16*)y, ldy, (const bf16*)g,
                  ldg, bias, b_dtype, weight, w_dtype, residual, (bf16*)act_out, dim, eps);
    } else {
        GI_REQUIRE(false, "gi_gate_norm_add: activation dtype %d", act_dtype);
    }
    return gi_check_launch("gi_gate_norm_add");
}

// ------------------------------------------------------------------ xIELU
template <typename T>
__global__ void xielu_kernel(const T* __restrict__ z, long long ldz, T* __restrict__ out, const void* __restrict__ pq,
                             int pq_dtype, int n_rows, int cols) {
    gi_pdl_start();
    const float a_pos = softplus_f(load_w(pq, pq_dtype, 0));
    const float a_neg = 0.5f + softplus_f(load_w(pq, pq_dtype, 1));
    const long long total = (long long)n_rows * cols;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / cols;
        const int c = (int)(i - r * cols);
        const float v = to_f32(z[r * ldz + c]);
        const float a = v > 0.f ? a_pos * v * v + 0.5f * v : a_neg * (expm1f(v) - v) + 0.5f * v;
        out[i] = from_f32<T>(a);
    }
}

extern "C" int gi_xielu(const void* z, long long ldz, void* out, int act_dtype, const void* pq, int pq_dtype,
                        int n_rows, int cols, void* stream) {
    GI_REQUIRE(n_rows >= 0 && cols > 0 && ldz >= cols, "gi_xielu: sizes");
    if (n_rows == 0) return 0;
    const long long total = (long long)n_rows * cols;
    const int blocks = (int)((total + 255) / 256 > 148 * 16 ? 148 * 16 : (total + 255) / 256);
    cudaStream_t s = (cudaStream_t)stream;
    if (act_dtype == GI_DTYPE_F32)
        gi_launch(xielu_kernel<float>, dim3(blocks), dim3(256), 0, s, (const float*)z, ldz, (float*)out, pq, pq_dtype, n_rows, cols);
    else if (act_dtype == GI_DTYPE_BF16)
        gi_launch(xielu_kernel<bf16>, dim3(blocks), dim3(256), 0, s, (const bf16*)z, ldz, (bf16*)out, pq, pq_dtype, n_rows, cols);
    else
        GI_REQUIRE(false, "gi_xielu: activation dtype %d", act_dtype);
    return gi_check_launch("gi_xielu");
}

// ------------------------------------------------------------------ group norm and gate of a read-out
// o float32 [n, groups * gs]; one block per (row, group); the result is also multiplied by `mul` and written to
// rows that lie ld_out apart (columns of a wider matrix).  weight[c % w_len]: w_len = gs (one weight for all
// groups) or groups * gs.  gate_kind 0: sigmoid(g), 1: silu(g); g has the columns of o, row stride ldg.
template <typename T>
__global__ void gated_group_rmsnorm_kernel(const float* __restrict__ o, const T* __restrict__ g, long long ldg,
                                           const void* __restrict__ weight, int w_dtype, int w_len,
                                           T* __restrict__ out, int groups, int gs, float eps, int gate_kind,
                                           float mul, long long ld_out) {
    gi_pdl_start();
    __shared__ float red[33];
    const size_t r = blockIdx.x;
    const int grp = blockIdx.y;
    const float* orow = o + (r * groups + grp) * gs;
    float ss = 0.f;
#pragma unroll 8
    for (int c = threadIdx.x; c < gs; c += blockDim.x) ss += orow[c] * orow[c];
    ss = block_sum(ss, red);
    const float inv = 1.f / sqrtf(ss / (float)gs + eps);
#pragma unroll 8
    for (int c = threadIdx.x; c < gs; c += blockDim.x) {
        const int col = grp * gs + c;
        const float z = to_f32(g[r * ldg + col]);
        const float gate = gate_kind == 0 ? sigmoid_f(z) : z * sigmoid_f(z);
        out[r * (size_t)ld_out + col] = from_f32<T>(orow[c] * inv * load_w(weight, w_dtype, col % w_len) * gate * mul);
    }
}

extern "C" int gi_gated_group_rmsnorm(const float* o, const void* g, long long ldg, const void* weight, int w_dtype,
                                      int w_len, void* out, int act_dtype, int n_rows, int groups, int gs, float eps,
                                      int gate_kind, float mul, long long ld_out, void* stream) {
    GI_REQUIRE(ld_out >= (long long)groups * gs, "gi_gated_group_rmsnorm: output rows shorter than the groups");
    GI_REQUIRE(n_rows >= 0 && groups > 0 && gs > 0 && groups <= 65535, "gi_gated_group_rmsnorm: sizes");
    GI_REQUIRE(w_len == gs || w_len == groups * gs, "gi_gated_group_rmsnorm: a weight of %d elements fits neither a "
               "group of %d nor the row of %d", w_len, gs, groups * gs);
    GI_REQUIRE(ldg >= (long long)groups * gs && (gate_kind == 0 || gate_kind == 1), "gi_gated_group_rmsnorm: gate");
    if (n_rows == 0) return 0;
    const int threads = gs >= 4096 ? 512 : (gs >= 1024 ? 256 : (gs >= 128 ? 128 : (gs > 32 ? 64 : 32)));
    cudaStream_t s = (cudaStream_t)stream;
    if (act_dtype == GI_DTYPE_F32)
        gi_launch(gated_group_rmsnorm_kernel<float>, dim3(n_rows, groups), dim3(threads), 0, s, o, (const float*)g, ldg,
                  weight, w_dtype, w_len, (float*)out, groups, gs, eps, gate_kind, mul, ld_out);
    else if (act_dtype == GI_DTYPE_BF16)
        gi_launch(gated_group_rmsnorm_kernel<bf16>, dim3(n_rows, groups), dim3(threads), 0, s, o, (const bf16*)g, ldg,
                  weight, w_dtype, w_len, (bf16*)out, groups, gs, eps, gate_kind, mul, ld_out);
    else
        GI_REQUIRE(false, "gi_gated_group_rmsnorm: activation dtype %d", act_dtype);
    return gi_check_launch("gi_gated_group_rmsnorm");
}
