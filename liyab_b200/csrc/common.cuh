// Shared helpers of the kernel library: status codes, the thread-local error
// message, element types and warp/block reductions.
//
// Every exported function returns a status in the reference's numbering
// (include/liyab/liyab_c_api.h:41-53) and leaves a message for lb_last_error(),
// the way the reference's C API guards every call and keeps a thread-local last
// error (src/c_api/liyab_c_api.cpp:34-58).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

enum lb_status : int {
    LB_OK = 0,
    LB_ERR_INVALID_ARGUMENT = 1,
    LB_ERR_UNSUPPORTED = 4,
    LB_ERR_BACKEND = 8,
    LB_ERR_INTERNAL = 10,
};

// Element types of tensors passed through the C interface.
enum lb_dtype : int {
    LB_F32 = 0,
    LB_BF16 = 1,
};

// Activations fused into a matrix product's epilogue.
enum lb_activation : int {
    LB_ACT_NONE = 0,
    LB_ACT_GELU_TANH = 1,
    LB_ACT_GELU_ERF = 2,
    // xIELU: z > 0 -> a z^2 + z/2, else b (exp(z) - 1 - z) + z/2 with a = softplus(p), b = 1/2 + softplus(q).  The two learned numbers
    // travel behind the bias: a product with this activation is given a bias of N + 2 floats, bias[N] = p and bias[N + 1] = q.
    LB_ACT_XIELU = 3,
    // The square of relu: max(z, 0)^2.
    LB_ACT_RELU2 = 4,
};

int lb_fail(int code, const char* fmt, ...);

#define LB_CHECK_ARG(cond, ...)                                      \
    do {                                                             \
        if (!(cond)) return lb_fail(LB_ERR_INVALID_ARGUMENT, __VA_ARGS__); \
    } while (0)

#define LB_CHECK_CUDA(expr)                                                                          \
    do {                                                                                             \
        cudaError_t err__ = (expr);                                                                  \
        if (err__ != cudaSuccess)                                                                    \
            return lb_fail(LB_ERR_BACKEND, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(err__), \
                           __FILE__, __LINE__);                                                      \
    } while (0)

#define LB_CHECK_LAUNCH() LB_CHECK_CUDA(cudaGetLastError())

// ---- launches that overlap the end of the kernel before ----
//
// A kernel launched through lb_launch_overlapped may be started while the kernel before it on the stream is still
// running (programmatic dependent launch): its blocks set up, ask for what does not depend on the kernel before
// (weights, block tables) and only then wait for it with lb_wait_for_predecessor(), which returns once that kernel
// has completed and its writes are visible.  Every thread of such a kernel passes lb_wait_for_predecessor() before
// it reads what an earlier kernel wrote or writes what an earlier kernel may still read.  The kernel before
// lets its successor start by lb_dependents_may_launch() (from all its blocks; without it the successor starts when
// it ends); a thread calls it only after its own lb_wait_for_predecessor(): let go before that, a step's later
// kernels ran ahead of data they needed (measured: wrong logits), whatever the reading of the instruction says.  In a kernel launched the ordinary way both are no-ops, and an ordinary launch after an overlapped one
// waits for the whole of it, as always.  lb_set_launch_overlap(0) makes every launch ordinary (measurements).
__device__ __forceinline__ void lb_dependents_may_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void lb_wait_for_predecessor() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

bool lb_launch_overlap_enabled(int kind = 0);

// cluster_x > 1: the grid's blocks form clusters of cluster_x blocks along x (gridDim.x a multiple of it).
template <typename... Params, typename... Args>
inline cudaError_t lb_launch_overlapped_cluster(int kind, int cluster_x, void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem,
                                                cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[2];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = lb_launch_overlap_enabled(kind) ? 1 : 0;
    config.attrs = attribute;
    config.numAttrs = 1;
    if (cluster_x > 1) {
        attribute[1].id = cudaLaunchAttributeClusterDimension;
        attribute[1].val.clusterDim.x = (unsigned)cluster_x;
        attribute[1].val.clusterDim.y = 1;
        attribute[1].val.clusterDim.z = 1;
        config.numAttrs = 2;
    }
    return cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
}

template <typename... Params, typename... Args>
inline cudaError_t lb_launch_overlapped_kind(int kind, void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                        Args... args) {
    return lb_launch_overlapped_cluster(kind, 1, kernel, grid, block, smem, stream, args...);
}

// The first key that the query at position `pos` sees.  `window` says which earlier keys are visible: 0 all of them; w > 0 the w
// latest (pos - w + 1 .. pos); w < 0 those of the query's own chunk of -w positions, chunks counted from position 0 of the sequence.
__host__ __device__ __forceinline__ int lb_first_visible(int pos, int window) {
    if (window > 0) return pos - window + 1 > 0 ? pos - window + 1 : 0;
    if (window < 0) return pos / (-window) * (-window);
    return 0;
}

// What a score loses by the distance between query and key, for heads that carry the pair (r1, r2): r1 ln(1 + r2 distance).
__device__ __forceinline__ float lb_distance_penalty(float r1, float r2, int distance) { return r1 * logf(fmaf(r2, (float)distance, 1.0f)); }

// A head's sink joins a finished softmax state: exp(sink) is added to the divisor, with no key and no value.  `m` is the state's running
// maximum and `sink` the head's number, both in the scale of the kernel's exponentials (base 2: sink * log2(e)); `l` becomes the new divisor
// and the result is the factor on the state's weighted values.
__device__ __forceinline__ float lb_sink_join_exp2(float sink, float m, float& l) {
    const float top = fmaxf(m, sink), f = exp2f(m - top);
    l = l * f + exp2f(sink - top);
    return f;
}
constexpr float kLbLog2e = 1.4426950408889634f;

__device__ __forceinline__ float lb_to_float(float v) { return v; }
__device__ __forceinline__ float lb_to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T lb_from_float(float v);
template <>
__device__ __forceinline__ float lb_from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 lb_from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float lb_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float lb_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  The
// order of additions is fixed by the block size alone.
__device__ __forceinline__ float lb_block_sum(float v, float* scratch /* >= 33 floats */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = (blockDim.x + 31) >> 5;
    v = lb_warp_sum(v);
    __syncthreads();  // scratch may still be read from a previous call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < n_warps ? scratch[lane] : 0.0f;
        t = lb_warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// GELU, tanh form: 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3)))
// (reference: src/core/transformer.cpp:125-130).
__device__ __forceinline__ float lb_gelu_tanh(float x) {
    const float k = 0.7978845608028654f;
    return 0.5f * x * (1.0f + tanhf(k * (x + 0.044715f * x * x * x)));
}

// GELU, exact form: 0.5 x (1 + erf(x / sqrt 2)) (reference: src/core/transformer.cpp:139-142).
__device__ __forceinline__ float lb_gelu_erf(float x) {
    return 0.5f * x * (1.0f + erff(x * 0.70710678118654752440f));
}

__device__ __forceinline__ float lb_softplus(float v) { return fmaxf(v, 0.0f) + log1pf(expf(-fabsf(v))); }
__device__ __forceinline__ float lb_xielu(float v, float a, float b) { return v > 0.0f ? fmaf(a * v, v, 0.5f * v) : fmaf(b, expm1f(v) - v, 0.5f * v); }

// The two factors of an activation with learned numbers (zeros for the others), read once by a thread before its epilogue.
struct lb_act_pair {
    float a, b;
};
__device__ __forceinline__ lb_act_pair lb_act_load(const float* bias, int N, int act) {
    lb_act_pair p{0.0f, 0.0f};
    if (act == LB_ACT_XIELU && bias != nullptr) {
        p.a = lb_softplus(__ldg(bias + N));
        p.b = 0.5f + lb_softplus(__ldg(bias + N + 1));
    }
    return p;
}

__device__ __forceinline__ float lb_activate(float x, int act) {
    if (act == LB_ACT_GELU_TANH) return lb_gelu_tanh(x);
    if (act == LB_ACT_GELU_ERF) return lb_gelu_erf(x);
    if (act == LB_ACT_RELU2) return x > 0.0f ? x * x : 0.0f;
    return x;
}

__device__ __forceinline__ float lb_activate(float x, int act, const lb_act_pair& p) {
    if (act == LB_ACT_XIELU) return lb_xielu(x, p.a, p.b);
    return lb_activate(x, act);
}

// The two halves of a gated feed-forward meet: act(g) * u.  Kinds: 0 sigmoid, 1 silu, 2 GELU (tanh form), 3 relu, and 4, the capped
// form with its two numbers (alpha, limit): g' = min(g, limit), u' = clamp(u, -limit, limit), g' sigmoid(alpha g') (u' + 1).
enum lb_gate_kind : int { LB_GATE_SIGMOID = 0, LB_GATE_SILU = 1, LB_GATE_GELU_TANH = 2, LB_GATE_RELU = 3, LB_GATE_CAPPED = 4 };
__device__ __forceinline__ float lb_gated_pair(float g, float u, int kind, float alpha, float limit) {
    if (kind == LB_GATE_CAPPED) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
        return g * (1.0f / (1.0f + expf(-alpha * g))) * (u + 1.0f);
    }
    const float sg = 1.0f / (1.0f + expf(-g));
    const float a = kind == LB_GATE_SILU ? g * sg : kind == LB_GATE_GELU_TANH ? lb_gelu_tanh(g) : kind == LB_GATE_RELU ? fmaxf(g, 0.0f) : sg;
    return a * u;
}

template <typename... Params, typename... Args>
inline cudaError_t lb_launch_overlapped(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    return lb_launch_overlapped_kind(0, kernel, grid, block, smem, stream, args...);
}
