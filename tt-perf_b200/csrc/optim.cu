// Optimiser updates as single fused passes over the parameters (HBM-bandwidth bound).
//   SGD : p <- p - lr * g                                  (2 reads + 1 write per element)
//   Adam: m, v, p updated in one pass; m and v are fp32    (p, g bf16: 2+2+4+4 bytes read, 2+4+4 written)
// A "multi-tensor" launch walks a table of up to 32 parameter tensors so that an optimiser step over a
// whole model is a handful of launches instead of one per tensor.
#include "common.cuh"
#include "gemm_common.cuh"

#include <algorithm>

namespace b200 {
namespace {

constexpr int kThreads = 256;
constexpr int kMaxTensors = 32;

struct TensorTable {
    void* p[kMaxTensors];
    const void* g[kMaxTensors];
    float* m[kMaxTensors];
    float* v[kMaxTensors];
    void* shadow[kMaxTensors];         // optional bf16 copy of an fp32 parameter, refreshed in the same pass
    long long n[kMaxTensors];
    long long start[kMaxTensors + 1];  // prefix sums of 8-element chunks
    int count;
};

struct AdamScalars {
    float lr, beta1, beta2, eps, inv_bias1, inv_bias2;
};

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

__device__ __forceinline__ int find_tensor(const TensorTable& t, long long chunk) {
    int lo = 0, hi = t.count - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (t.start[mid] <= chunk) lo = mid; else hi = mid - 1;
    }
    return lo;
}

// p_f32 / g_f32: storage type of parameters and gradients (0 = bf16, 1 = fp32).
template <bool ADAM>
__global__ void __launch_bounds__(kThreads) optim_kernel(const TensorTable t, const AdamScalars s, int p_f32, int g_f32) {
    const long long total = t.start[t.count];
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long chunk = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; chunk < total; chunk += stride) {
        const int ti = find_tensor(t, chunk);
        const long long base = (chunk - t.start[ti]) * 8;
        const long long n = t.n[ti];
        const int cnt = static_cast<int>(min(8ll, n - base));
        float pv[8], gv[8];
        const bool full = cnt == 8;
        // parameters and gradients
        if (p_f32) {
            const float* pp = static_cast<const float*>(t.p[ti]) + base;
            for (int i = 0; i < cnt; ++i) pv[i] = pp[i];
        } else {
            const __nv_bfloat16* pp = static_cast<const __nv_bfloat16*>(t.p[ti]) + base;
            if (full && ((reinterpret_cast<uintptr_t>(pp) & 15u) == 0)) {
                unpack8(*reinterpret_cast<const uint4*>(pp), pv);
            } else {
                for (int i = 0; i < cnt; ++i) pv[i] = __bfloat162float(pp[i]);
            }
        }
        if (g_f32) {
            const float* gp = static_cast<const float*>(t.g[ti]) + base;
            for (int i = 0; i < cnt; ++i) gv[i] = gp[i];
        } else {
            const __nv_bfloat16* gp = static_cast<const __nv_bfloat16*>(t.g[ti]) + base;
            if (full && ((reinterpret_cast<uintptr_t>(gp) & 15u) == 0)) {
                unpack8(*reinterpret_cast<const uint4*>(gp), gv);
            } else {
                for (int i = 0; i < cnt; ++i) gv[i] = __bfloat162float(gp[i]);
            }
        }
        if (ADAM) {
            float* mp = t.m[ti] + base;
            float* vp = t.v[ti] + base;
            float mv[8], vv[8];
            const bool mvec = full && ((reinterpret_cast<uintptr_t>(mp) & 15u) == 0) &&
                              ((reinterpret_cast<uintptr_t>(vp) & 15u) == 0);
            if (mvec) {
                const float4 m0 = reinterpret_cast<const float4*>(mp)[0], m1 = reinterpret_cast<const float4*>(mp)[1];
                const float4 v0 = reinterpret_cast<const float4*>(vp)[0], v1 = reinterpret_cast<const float4*>(vp)[1];
                mv[0] = m0.x; mv[1] = m0.y; mv[2] = m0.z; mv[3] = m0.w; mv[4] = m1.x; mv[5] = m1.y; mv[6] = m1.z; mv[7] = m1.w;
                vv[0] = v0.x; vv[1] = v0.y; vv[2] = v0.z; vv[3] = v0.w; vv[4] = v1.x; vv[5] = v1.y; vv[6] = v1.z; vv[7] = v1.w;
            } else {
                for (int i = 0; i < cnt; ++i) {
                    mv[i] = mp[i];
                    vv[i] = vp[i];
                }
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                if (i < cnt) {
                    mv[i] = s.beta1 * mv[i] + (1.0f - s.beta1) * gv[i];
                    vv[i] = s.beta2 * vv[i] + (1.0f - s.beta2) * gv[i] * gv[i];
                    pv[i] -= s.lr * (mv[i] * s.inv_bias1) / (sqrtf(vv[i] * s.inv_bias2) + s.eps);
                }
            }
            if (mvec) {
                reinterpret_cast<float4*>(mp)[0] = make_float4(mv[0], mv[1], mv[2], mv[3]);
                reinterpret_cast<float4*>(mp)[1] = make_float4(mv[4], mv[5], mv[6], mv[7]);
                reinterpret_cast<float4*>(vp)[0] = make_float4(vv[0], vv[1], vv[2], vv[3]);
                reinterpret_cast<float4*>(vp)[1] = make_float4(vv[4], vv[5], vv[6], vv[7]);
            } else {
                for (int i = 0; i < cnt; ++i) {
                    mp[i] = mv[i];
                    vp[i] = vv[i];
                }
            }
        } else {
            for (int i = 0; i < cnt; ++i) pv[i] -= s.lr * gv[i];
        }
        if (t.shadow[ti] != nullptr) {
            __nv_bfloat16* sp = static_cast<__nv_bfloat16*>(t.shadow[ti]) + base;
            if (full && ((reinterpret_cast<uintptr_t>(sp) & 15u) == 0)) {
                *reinterpret_cast<uint4*>(sp) = make_uint4(pack_bf16x2(pv[0], pv[1]), pack_bf16x2(pv[2], pv[3]),
                                                           pack_bf16x2(pv[4], pv[5]), pack_bf16x2(pv[6], pv[7]));
            } else {
                for (int i = 0; i < cnt; ++i) sp[i] = __float2bfloat16_rn(pv[i]);
            }
        }
        if (p_f32) {
            float* pp = static_cast<float*>(t.p[ti]) + base;
            for (int i = 0; i < cnt; ++i) pp[i] = pv[i];
        } else {
            __nv_bfloat16* pp = static_cast<__nv_bfloat16*>(t.p[ti]) + base;
            if (full && ((reinterpret_cast<uintptr_t>(pp) & 15u) == 0)) {
                *reinterpret_cast<uint4*>(pp) = make_uint4(pack_bf16x2(pv[0], pv[1]), pack_bf16x2(pv[2], pv[3]),
                                                           pack_bf16x2(pv[4], pv[5]), pack_bf16x2(pv[6], pv[7]));
            } else {
                for (int i = 0; i < cnt; ++i) pp[i] = __float2bfloat16_rn(pv[i]);
            }
        }
    }
}

template <bool ADAM>
int run_optim(b200_ctx* ctx, const char* who, int64_t count, void* const* params, const void* const* grads, float* const* m,
              float* const* v, void* const* shadow, const int64_t* sizes, int p_dtype, int g_dtype, const AdamScalars& s, void* stream) {
    B200_REQUIRE(ctx != nullptr, "%s: ctx is NULL", who);
    B200_REQUIRE(count >= 0, "%s: negative tensor count", who);
    B200_REQUIRE((p_dtype == B200_BF16 || p_dtype == B200_F32) && (g_dtype == B200_BF16 || g_dtype == B200_F32),
                 "%s: parameter and gradient dtypes must be BF16 or F32", who);
    if (count == 0) return B200_OK;
    B200_REQUIRE(params && grads && sizes, "%s: NULL table", who);
    if (ADAM) B200_REQUIRE(m && v, "%s: NULL moment table", who);
    DeviceScope scope(ctx->device);
    cudaStream_t st = ctx->pick(stream);
    for (int64_t first = 0; first < count; first += kMaxTensors) {
        TensorTable t{};
        t.count = 0;
        t.start[0] = 0;
        for (int64_t i = first; i < std::min<int64_t>(count, first + kMaxTensors); ++i) {
            B200_REQUIRE(sizes[i] >= 0, "%s: negative size for tensor %lld", who, (long long)i);
            if (sizes[i] == 0) continue;
            B200_REQUIRE(params[i] && grads[i], "%s: NULL parameter or gradient %lld", who, (long long)i);
            if (ADAM) B200_REQUIRE(m[i] && v[i], "%s: NULL moment buffer %lld", who, (long long)i);
            const int k = t.count++;
            t.p[k] = params[i];
            t.g[k] = grads[i];
            t.m[k] = ADAM ? m[i] : nullptr;
            t.v[k] = ADAM ? v[i] : nullptr;
            t.shadow[k] = shadow ? shadow[i] : nullptr;
            t.n[k] = sizes[i];
            t.start[k + 1] = t.start[k] + (sizes[i] + 7) / 8;
        }
        if (t.count == 0) continue;
        const long long chunks = t.start[t.count];
        const int blocks = static_cast<int>(std::max<long long>(1, std::min<long long>((chunks + kThreads - 1) / kThreads,
                                                                                       ctx->sm_count * 16ll)));
        optim_kernel<ADAM><<<blocks, kThreads, 0, st>>>(t, s, p_dtype == B200_F32, g_dtype == B200_F32);
        B200_CUDA_TRY(cudaGetLastError());
    }
    return B200_OK;
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

int b200_sgd_step(b200_ctx* ctx, int64_t count, void* const* params, const void* const* grads, void* const* shadow_bf16,
                  const int64_t* sizes, int p_dtype, int g_dtype, float lr, void* stream) {
    AdamScalars s{};
    s.lr = lr;
    return run_optim<false>(ctx, "b200_sgd_step", count, params, grads, nullptr, nullptr, shadow_bf16, sizes, p_dtype,
                            g_dtype, s, stream);
}

int b200_adam_step(b200_ctx* ctx, int64_t count, void* const* params, const void* const* grads, float* const* m,
                   float* const* v, void* const* shadow_bf16, const int64_t* sizes, int p_dtype, int g_dtype, float lr, float beta1, float beta2,
                   float eps, int64_t step, void* stream) {
    B200_REQUIRE(step >= 1, "b200_adam_step: step counts from 1 (got %lld)", (long long)step);
    B200_REQUIRE(lr > 0.0f && eps > 0.0f, "b200_adam_step: lr and eps must be > 0");
    B200_REQUIRE(beta1 > 0.0f && beta1 < 1.0f && beta2 > 0.0f && beta2 < 1.0f, "b200_adam_step: betas must be in (0, 1)");
    AdamScalars s{};
    s.lr = lr;
    s.beta1 = beta1;
    s.beta2 = beta2;
    s.eps = eps;
    s.inv_bias1 = static_cast<float>(1.0 / (1.0 - pow(static_cast<double>(beta1), static_cast<double>(step))));
    s.inv_bias2 = static_cast<float>(1.0 / (1.0 - pow(static_cast<double>(beta2), static_cast<double>(step))));
    return run_optim<true>(ctx, "b200_adam_step", count, params, grads, m, v, shadow_bf16, sizes, p_dtype, g_dtype, s,
                           stream);
}

}  // extern "C"
