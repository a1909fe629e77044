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
    const float* dev_bias;  // non-null: the two bias-correction factors live in device memory (see adam_advance_kernel)
};

// Device-resident step state of an optimiser whose step may be replayed from a recorded trace: the step number and
// the bias-correction factors 1 / (1 - beta^t) derived from it. Kernel arguments are frozen when a trace is recorded;
// memory is not, so a replayed step advances like an eager one.
struct AdamDeviceState {
    long long step;
    float inv_bias1, inv_bias2;
};

__global__ void adam_advance_kernel(AdamDeviceState* st, float beta1, float beta2) {
    const long long t = st->step + 1;
    st->step = t;
    st->inv_bias1 = static_cast<float>(1.0 / (1.0 - pow(static_cast<double>(beta1), static_cast<double>(t))));
    st->inv_bias2 = static_cast<float>(1.0 / (1.0 - pow(static_cast<double>(beta2), static_cast<double>(t))));
}

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

__device__ __forceinline__ float adam_update(float p, float g, float& m, float& v, const AdamScalars& s) {
    m = s.beta1 * m + (1.0f - s.beta1) * g;
    v = s.beta2 * v + (1.0f - s.beta2) * g * g;
    return p - __fdividef(s.lr * (m * s.inv_bias1), sqrtf(v * s.inv_bias2) + s.eps);
}

template <bool F32>
__device__ __forceinline__ float load_elem(const void* base, long long i) {
    return F32 ? static_cast<const float*>(base)[i] : __bfloat162float(static_cast<const __nv_bfloat16*>(base)[i]);
}
template <bool F32>
__device__ __forceinline__ void load8(const void* base, long long i, float (&f)[8]) {
    if (F32) {
        const float4 a = *reinterpret_cast<const float4*>(static_cast<const float*>(base) + i);
        const float4 b = *reinterpret_cast<const float4*>(static_cast<const float*>(base) + i + 4);
        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    } else {
        unpack8(*reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(base) + i), f);
    }
}
template <bool F32>
__device__ __forceinline__ void store8(void* base, long long i, const float (&f)[8]) {
    if (F32) {
        float* p = static_cast<float*>(base) + i;
        *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
        *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
    } else {
        *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(base) + i) =
            make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
    }
}

// blockIdx.y selects the tensor (uniform per CTA); blockIdx.x strides over its 8-element chunks. CTAs beyond a small
// tensor's last chunk fall straight through. Full, 16-byte aligned chunks use vector accesses with everything in
// registers; the ragged tail (and unaligned tensors) go element by element.
template <bool ADAM, bool P_F32, bool G_F32>
__global__ void __launch_bounds__(kThreads) optim_kernel(const TensorTable t, const AdamScalars s_in) {
    AdamScalars s = s_in;
    if (ADAM && s.dev_bias != nullptr) {
        s.inv_bias1 = s.dev_bias[0];
        s.inv_bias2 = s.dev_bias[1];
    }
    const int ti = blockIdx.y;
    const long long n = t.n[ti];
    void* const pp = t.p[ti];
    const void* const gp = t.g[ti];
    float* const mp = t.m[ti];
    float* const vp = t.v[ti];
    void* const sp = t.shadow[ti];
    const uintptr_t bits = reinterpret_cast<uintptr_t>(pp) | reinterpret_cast<uintptr_t>(gp) |
                           reinterpret_cast<uintptr_t>(mp) | reinterpret_cast<uintptr_t>(vp) |
                           reinterpret_cast<uintptr_t>(sp);
    const bool aligned = (bits & 15u) == 0;
    const long long nvec = aligned ? n / 8 : 0;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    const long long tid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    for (long long chunk = tid; chunk < nvec; chunk += stride) {
        const long long base = chunk * 8;
        float pv[8], gv[8];
        load8<P_F32>(pp, base, pv);
        load8<G_F32>(gp, base, gv);
        if (ADAM) {
            float mv[8], vv[8];
            load8<true>(mp, base, mv);
            load8<true>(vp, base, vv);
#pragma unroll
            for (int i = 0; i < 8; ++i) pv[i] = adam_update(pv[i], gv[i], mv[i], vv[i], s);
            store8<true>(mp, base, mv);
            store8<true>(vp, base, vv);
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) pv[i] -= s.lr * gv[i];
        }
        store8<P_F32>(pp, base, pv);
        if (sp != nullptr) store8<false>(sp, base, pv);
    }
    for (long long i = nvec * 8 + tid; i < n; i += stride) {
        float p = load_elem<P_F32>(pp, i);
        const float g = load_elem<G_F32>(gp, i);
        if (ADAM) {
            float m = mp[i], v = vp[i];
            p = adam_update(p, g, m, v, s);
            mp[i] = m;
            vp[i] = v;
        } else {
            p -= s.lr * g;
        }
        if (P_F32)
            static_cast<float*>(pp)[i] = p;
        else
            static_cast<__nv_bfloat16*>(pp)[i] = __float2bfloat16_rn(p);
        if (sp != nullptr) static_cast<__nv_bfloat16*>(sp)[i] = __float2bfloat16_rn(p);
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
        long long largest = 0;
        for (int k = 0; k < t.count; ++k) largest = std::max(largest, (t.n[k] + 7) / 8);
        const int blocks = static_cast<int>(std::max<long long>(1, std::min<long long>((largest + kThreads - 1) / kThreads,
                                                                                       ctx->sm_count * 8ll)));
        dim3 grid(static_cast<unsigned>(blocks), static_cast<unsigned>(t.count));
        const bool pf = p_dtype == B200_F32, gf = g_dtype == B200_F32;
        if (pf && gf)
            optim_kernel<ADAM, true, true><<<grid, kThreads, 0, st>>>(t, s);
        else if (pf)
            optim_kernel<ADAM, true, false><<<grid, kThreads, 0, st>>>(t, s);
        else if (gf)
            optim_kernel<ADAM, false, true><<<grid, kThreads, 0, st>>>(t, s);
        else
            optim_kernel<ADAM, false, false><<<grid, kThreads, 0, st>>>(t, s);
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

int b200_adam_step_device(b200_ctx* ctx, int64_t count, void* const* params, const void* const* grads, float* const* m,
                          float* const* v, void* const* shadow_bf16, const int64_t* sizes, int p_dtype, int g_dtype, float lr,
                          float beta1, float beta2, float eps, void* d_state16, int advance, void* stream) {
    B200_REQUIRE(ctx != nullptr, "b200_adam_step_device: ctx is NULL");
    B200_REQUIRE(d_state16 != nullptr && (reinterpret_cast<uintptr_t>(d_state16) & 7u) == 0,
                 "b200_adam_step_device: d_state16 must be an 8-byte aligned device buffer of 16 bytes");
    B200_REQUIRE(lr > 0.0f && eps > 0.0f, "b200_adam_step_device: lr and eps must be > 0");
    B200_REQUIRE(beta1 > 0.0f && beta1 < 1.0f && beta2 > 0.0f && beta2 < 1.0f, "b200_adam_step_device: betas must be in (0, 1)");
    AdamDeviceState* st = static_cast<AdamDeviceState*>(d_state16);
    static_assert(sizeof(AdamDeviceState) == 16, "device step state is 16 bytes");
    if (advance) {
        DeviceScope scope(ctx->device);
        adam_advance_kernel<<<1, 1, 0, ctx->pick(stream)>>>(st, beta1, beta2);
        B200_CUDA_TRY(cudaGetLastError());
    }
    AdamScalars s{};
    s.lr = lr;
    s.beta1 = beta1;
    s.beta2 = beta2;
    s.eps = eps;
    s.dev_bias = &st->inv_bias1;
    return run_optim<true>(ctx, "b200_adam_step_device", count, params, grads, m, v, shadow_bf16, sizes, p_dtype, g_dtype, s,
                           stream);
}

}  // extern "C"
