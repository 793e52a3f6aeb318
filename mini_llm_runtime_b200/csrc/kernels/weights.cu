// Kernels of the weight loader: the portable normal-number generator of the
// random-weights mode, and the finiteness check every uploaded tensor passes.
//
// The generator restates `weights/portable_random.py` step for step: 64-bit integer mixing,
// then Box-Muller in double precision with `ln` and `cos` written out as series.  Every
// floating-point step is an explicit round-to-nearest intrinsic (`__dmul_rn`, `__dadd_rn`,
// `__ddiv_rn`, `__dsqrt_rn`), so the compiler fuses nothing and the host's numpy version, which
// performs the same IEEE operations one by one, gives the same bits.
//
// The finiteness check is the reference's rule that a tensor with a NaN or an infinity is
// refused (src/minillm/cuda/storage.cpp:314-321), done on the device after the upload.
#include "common.cuh"

namespace {

constexpr unsigned long long kGolden = 0x9E3779B97F4A7C15ull;

__device__ __forceinline__ unsigned long long mix64(unsigned long long x) {
    x ^= x >> 30;
    x *= 0xBF58476D1CE4E5B9ull;
    x ^= x >> 27;
    x *= 0x94D049BB133111EBull;
    x ^= x >> 31;
    return x;
}

__device__ __forceinline__ double mul(double a, double b) { return __dmul_rn(a, b); }
__device__ __forceinline__ double add(double a, double b) { return __dadd_rn(a, b); }

__device__ double series_ln(double u) {
    int e;
    double m = frexp(u, &e);                       // exact: u = m 2^e, m in [0.5, 1)
    if (m < 0.7071067811865476) {
        m = mul(m, 2.0);
        e -= 1;
    }
    const double s = __ddiv_rn(add(m, -1.0), add(m, 1.0));
    const double s2 = mul(s, s);
    double poly = 1.0 / 21.0;
    poly = add(mul(poly, s2), 1.0 / 19.0);
    poly = add(mul(poly, s2), 1.0 / 17.0);
    poly = add(mul(poly, s2), 1.0 / 15.0);
    poly = add(mul(poly, s2), 1.0 / 13.0);
    poly = add(mul(poly, s2), 1.0 / 11.0);
    poly = add(mul(poly, s2), 1.0 / 9.0);
    poly = add(mul(poly, s2), 1.0 / 7.0);
    poly = add(mul(poly, s2), 1.0 / 5.0);
    poly = add(mul(poly, s2), 1.0 / 3.0);
    poly = add(mul(poly, s2), 1.0 / 1.0);
    return add(mul(static_cast<double>(e), 0.6931471805599453), mul(mul(2.0, s), poly));
}

__device__ double series_cos_turns(double t) {     // cos(2 pi t), t in [0, 1)
    const double a = mul(t, 4.0);
    const double j = floor(add(a, 0.5));
    const double theta = mul(add(a, -j), 1.5707963267948966);
    const double t2 = mul(theta, theta);
    double c = 1.0 / 20922789888000.0;              // 16!
    c = add(mul(c, t2), -1.0 / 87178291200.0);      // 14!
    c = add(mul(c, t2), 1.0 / 479001600.0);         // 12!
    c = add(mul(c, t2), -1.0 / 3628800.0);          // 10!
    c = add(mul(c, t2), 1.0 / 40320.0);             // 8!
    c = add(mul(c, t2), -1.0 / 720.0);              // 6!
    c = add(mul(c, t2), 1.0 / 24.0);                // 4!
    c = add(mul(c, t2), -1.0 / 2.0);                // 2!
    c = add(mul(c, t2), 1.0);
    double s = 1.0 / 355687428096000.0;             // 17!
    s = add(mul(s, t2), -1.0 / 1307674368000.0);    // 15!
    s = add(mul(s, t2), 1.0 / 6227020800.0);        // 13!
    s = add(mul(s, t2), -1.0 / 39916800.0);         // 11!
    s = add(mul(s, t2), 1.0 / 362880.0);            // 9!
    s = add(mul(s, t2), -1.0 / 5040.0);             // 7!
    s = add(mul(s, t2), 1.0 / 120.0);               // 5!
    s = add(mul(s, t2), -1.0 / 6.0);                // 3!
    s = mul(add(mul(s, t2), 1.0), theta);
    const int quarter = static_cast<int>(static_cast<long long>(j)) & 3;
    return quarter == 0 ? c : quarter == 1 ? -s : quarter == 2 ? -c : s;
}

template <typename T>
__global__ void normal_fill_kernel(T* __restrict__ out, long long count, unsigned long long key, double std, int one_plus) {
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += stride) {
        const unsigned long long c = key + (static_cast<unsigned long long>(i) * 2ull) * kGolden;
        const unsigned long long a = mix64(c), b = mix64(c + kGolden);
        const double u1 = mul(static_cast<double>((a >> 11) + 1ull), 0x1p-53);
        const double u2 = mul(static_cast<double>(b >> 11), 0x1p-53);
        const double z = mul(__dsqrt_rn(mul(-2.0, series_ln(u1))), series_cos_turns(u2));
        double v = mul(z, std);
        if (one_plus) v = add(v, 1.0);
        mlr_store(out, static_cast<size_t>(i), __double2float_rn(v));
    }
}

template <typename T>
__global__ void finite_check_kernel(const T* __restrict__ data, long long count, int* __restrict__ flag) {
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    bool bad = false;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += stride) {
        const float v = mlr_load(data, static_cast<size_t>(i));
        bad |= !(fabsf(v) <= 3.402823466e+38f);     // false for NaN and for either infinity
    }
    if (__any_sync(0xffffffffu, bad) && (threadIdx.x & 31) == 0) *flag = 1;
}

int grid_for(long long count) {
    return mlr_grid_stride_blocks(static_cast<size_t>((count + 255) / 256), 32);
}

}  // namespace

// out[i] = N(0, std^2) (or 1 + N(0, std^2)) for element i of the tensor whose key is `key`
// (`tensor_key(seed, name)` of weights/portable_random.py), rounded once to float32 and, for a
// bfloat16 output, once more to bfloat16.
MLR_API int mlr_normal_fill(void* out, int out_bf16, long long count, unsigned long long key, double std, int one_plus,
                            void* stream) {
    MLR_REQUIRE(count >= 0 && std >= 0.0, "normal_fill: bad count %lld or deviation %g", count, std);
    if (count == 0) return 0;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (out_bf16)
        normal_fill_kernel<<<grid_for(count), 256, 0, s>>>(static_cast<__nv_bfloat16*>(out), count, key, std, one_plus);
    else
        normal_fill_kernel<<<grid_for(count), 256, 0, s>>>(static_cast<float*>(out), count, key, std, one_plus);
    return mlr_launched("normal_fill");
}

// *flag = 1 if any of the `count` elements is a NaN or an infinity (the flag is left alone otherwise).
MLR_API int mlr_finite_check(const void* data, int is_bf16, long long count, int* flag, void* stream) {
    MLR_REQUIRE(count >= 0, "finite_check: bad count %lld", count);
    if (count == 0) return 0;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (is_bf16)
        finite_check_kernel<<<grid_for(count), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(data), count, flag);
    else
        finite_check_kernel<<<grid_for(count), 256, 0, s>>>(static_cast<const float*>(data), count, flag);
    return mlr_launched("finite_check");
}
