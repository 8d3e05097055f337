// Seeded synthetic weights, generated and quantised on the GPU in ggml block layout.
// The reference loads GGUF files; benchmarks here have no model files, so tensors are drawn from
// N(0, std) with a counter-based generator (value depends only on seed and element index) and
// packed with a min/max affine fit per sub-block.  Only the decoders are pinned to ggml; any
// valid block is a legitimate input.
#include "tiles.cuh"

namespace dfl {

dfl_status use_device(int device);

__device__ __forceinline__ uint64_t mix64(uint64_t z) {
    z += 0x9e3779b97f4a7c15ull;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}
// standard normal for element `idx` (Box-Muller on a hashed counter)
__device__ __forceinline__ float normal_at(uint64_t seed, uint64_t idx) {
    const uint64_t h = mix64(seed ^ mix64(idx));
    const float u1 = ((uint32_t)(h >> 40) + 1.0f) * (1.0f / 16777217.0f);  // (0, 1)
    const float u2 = (uint32_t)((h >> 8) & 0xffffffu) * (1.0f / 16777216.0f);
    return sqrtf(-2.0f * __logf(u1)) * __cosf(6.28318530718f * u2);
}
__device__ __forceinline__ void put16(uint8_t* p, uint16_t v) { p[0] = (uint8_t)v; p[1] = (uint8_t)(v >> 8); }

// one thread per 256-weight super-block
template <int LEVELS>  // 15 = Q4_K, 31 = Q5_K
__global__ void synth_k45_kernel(uint8_t* __restrict__ dst, uint64_t n_blocks, uint64_t seed, float std_dev) {
    const uint64_t b = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= n_blocks) return;
    constexpr int BYTES = LEVELS == 15 ? 144 : 176;
    uint8_t* blk = dst + b * BYTES;
    float scl[8], mns[8], max_s = 0.f, max_m = 0.f;
    for (int j = 0; j < 8; ++j) {
        float lo = 0.f, hi = -INFINITY;
        for (int l = 0; l < 32; ++l) {
            const float x = std_dev * normal_at(seed, b * 256 + 32 * j + l);
            lo = fminf(lo, x);
            hi = fmaxf(hi, x);
        }
        hi = fmaxf(hi, lo);
        scl[j] = (hi - lo) / (float)LEVELS;
        mns[j] = -lo;
        max_s = fmaxf(max_s, scl[j]);
        max_m = fmaxf(max_m, mns[j]);
    }
    const __half dh = __float2half_rn(max_s / 63.f), mh = __float2half_rn(max_m / 63.f);
    const float d = __half2float(dh), dmin = __half2float(mh);
    uint8_t sc[8], mn[8];
    for (int j = 0; j < 8; ++j) {
        sc[j] = (uint8_t)min(63, max(0, d > 0.f ? __float2int_rn(scl[j] / d) : 0));
        mn[j] = (uint8_t)min(63, max(0, dmin > 0.f ? __float2int_rn(mns[j] / dmin) : 0));
    }
    put16(blk, __half_as_ushort(dh));
    put16(blk + 2, __half_as_ushort(mh));
    for (int j = 0; j < 4; ++j) {
        blk[4 + j] = (uint8_t)((sc[j] & 63) | ((sc[j + 4] >> 4) << 6));
        blk[8 + j] = (uint8_t)((mn[j] & 63) | ((mn[j + 4] >> 4) << 6));
        blk[12 + j] = (uint8_t)((sc[j + 4] & 0x0f) | ((mn[j + 4] & 0x0f) << 4));
    }
    uint8_t* qh = blk + 16;
    uint8_t* qs = blk + (LEVELS == 15 ? 16 : 48);
    if (LEVELS == 31)
        for (int l = 0; l < 32; ++l) qh[l] = 0;
    for (int c = 0; c < 4; ++c) {
        const float ds0 = d * sc[2 * c], dm0 = dmin * mn[2 * c], ds1 = d * sc[2 * c + 1], dm1 = dmin * mn[2 * c + 1];
        for (int l = 0; l < 32; ++l) {
            const float x0 = std_dev * normal_at(seed, b * 256 + 64 * c + l);
            const float x1 = std_dev * normal_at(seed, b * 256 + 64 * c + 32 + l);
            const int q0 = min(LEVELS, max(0, ds0 > 0.f ? __float2int_rn((x0 + dm0) / ds0) : 0));
            const int q1 = min(LEVELS, max(0, ds1 > 0.f ? __float2int_rn((x1 + dm1) / ds1) : 0));
            qs[32 * c + l] = (uint8_t)((q0 & 15) | ((q1 & 15) << 4));
            if (LEVELS == 31) qh[l] |= (uint8_t)((((q0 >> 4) & 1) << (2 * c)) | (((q1 >> 4) & 1) << (2 * c + 1)));
        }
    }
}

__global__ void synth_q6k_kernel(uint8_t* __restrict__ dst, uint64_t n_blocks, uint64_t seed, float std_dev) {
    const uint64_t b = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= n_blocks) return;
    uint8_t* blk = dst + b * 210;
    float scl[16], max_s = 0.f;
    for (int j = 0; j < 16; ++j) {
        float amax = 0.f;
        for (int l = 0; l < 16; ++l) amax = fmaxf(amax, fabsf(std_dev * normal_at(seed, b * 256 + 16 * j + l)));
        scl[j] = amax / 31.f;
        max_s = fmaxf(max_s, scl[j]);
    }
    const __half dh = __float2half_rn(max_s / 127.f);
    const float d = __half2float(dh);
    int8_t sc[16];
    for (int j = 0; j < 16; ++j) sc[j] = (int8_t)min(127, max(-128, d > 0.f ? __float2int_rn(scl[j] / d) : 0));
    auto quant = [&](int i) -> uint32_t {
        const float ds = d * (float)sc[i >> 4];
        const float x = std_dev * normal_at(seed, b * 256 + i);
        return (uint32_t)(min(31, max(-32, ds != 0.f ? __float2int_rn(x / ds) : 0)) + 32);
    };
    for (int n = 0; n < 2; ++n)
        for (int l = 0; l < 32; ++l) {
            const uint32_t q1 = quant(128 * n + l), q2 = quant(128 * n + 32 + l), q3 = quant(128 * n + 64 + l), q4 = quant(128 * n + 96 + l);
            blk[64 * n + l] = (uint8_t)((q1 & 15) | ((q3 & 15) << 4));
            blk[64 * n + 32 + l] = (uint8_t)((q2 & 15) | ((q4 & 15) << 4));
            blk[128 + 32 * n + l] = (uint8_t)((q1 >> 4) | ((q2 >> 4) << 2) | ((q3 >> 4) << 4) | ((q4 >> 4) << 6));
        }
    for (int j = 0; j < 16; ++j) blk[192 + j] = (uint8_t)sc[j];
    put16(blk + 208, __half_as_ushort(dh));
}

__global__ void synth_q80_kernel(uint8_t* __restrict__ dst, uint64_t n_blocks, uint64_t seed, float std_dev) {
    const uint64_t b = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= n_blocks) return;
    uint8_t* blk = dst + b * 34;
    float amax = 0.f;
    for (int l = 0; l < 32; ++l) amax = fmaxf(amax, fabsf(std_dev * normal_at(seed, b * 32 + l)));
    const __half dh = __float2half_rn(amax / 127.f);
    const float d = __half2float(dh);
    put16(blk, __half_as_ushort(dh));
    for (int l = 0; l < 32; ++l)
        blk[2 + l] = (uint8_t)(int8_t)min(127, max(-127, d > 0.f ? __float2int_rn(std_dev * normal_at(seed, b * 32 + l) / d) : 0));
}

__global__ void synth_plain_kernel(int dtype, uint8_t* __restrict__ dst, uint64_t n, uint64_t seed, float std_dev) {
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float x = std_dev * normal_at(seed, i);
    if (dtype == DFL_F32) reinterpret_cast<float*>(dst)[i] = x;
    else if (dtype == DFL_F16) reinterpret_cast<__half*>(dst)[i] = __float2half_rn(x);
    else reinterpret_cast<__nv_bfloat16*>(dst)[i] = __float2bfloat16_rn(x);
}

}  // namespace dfl

using namespace dfl;

extern "C" {

dfl_status dfl_synth_tensor(int32_t device, int32_t dtype, uint64_t n_in, uint64_t n_out, uint64_t seed, float std_dev, void** dev_ptr,
                            uint64_t* n_bytes) {
    if (!dev_ptr || !n_bytes) return fail(DFL_ERR_BAD_ARG, "synth_tensor: null argument");
    *dev_ptr = nullptr;
    DFL_CHECK(use_device(device));
    const uint64_t n = n_in * n_out;
    uint64_t bytes = 0, blocks = 0;
    switch (dtype) {
        case DFL_F32: bytes = n * 4; break;
        case DFL_F16:
        case DFL_BF16: bytes = n * 2; break;
        case DFL_Q8_0: if (n_in % 32) return fail(DFL_ERR_BAD_SHAPE, "synth_tensor: row not block aligned"); blocks = n / 32; bytes = blocks * 34; break;
        case DFL_Q4_K: if (n_in % 256) return fail(DFL_ERR_BAD_SHAPE, "synth_tensor: row not block aligned"); blocks = n / 256; bytes = blocks * 144; break;
        case DFL_Q5_K: if (n_in % 256) return fail(DFL_ERR_BAD_SHAPE, "synth_tensor: row not block aligned"); blocks = n / 256; bytes = blocks * 176; break;
        case DFL_Q6_K: if (n_in % 256) return fail(DFL_ERR_BAD_SHAPE, "synth_tensor: row not block aligned"); blocks = n / 256; bytes = blocks * 210; break;
        default: return fail(DFL_ERR_UNSUPPORTED, "synth_tensor: dtype");
    }
    uint8_t* p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) return fail(DFL_ERR_OOM, "synth_tensor: cudaMalloc failed");
    const unsigned tb = 128;
    switch (dtype) {
        case DFL_Q4_K: synth_k45_kernel<15><<<(unsigned)((blocks + tb - 1) / tb), tb>>>(p, blocks, seed, std_dev); break;
        case DFL_Q5_K: synth_k45_kernel<31><<<(unsigned)((blocks + tb - 1) / tb), tb>>>(p, blocks, seed, std_dev); break;
        case DFL_Q6_K: synth_q6k_kernel<<<(unsigned)((blocks + tb - 1) / tb), tb>>>(p, blocks, seed, std_dev); break;
        case DFL_Q8_0: synth_q80_kernel<<<(unsigned)((blocks + tb - 1) / tb), tb>>>(p, blocks, seed, std_dev); break;
        default: synth_plain_kernel<<<(unsigned)((n + 255) / 256), 256>>>(dtype, p, n, seed, std_dev); break;
    }
    count_launch();
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        cudaFree(p);
        return fail(DFL_ERR_CUDA, std::string("synth_tensor: ") + cudaGetErrorString(e));
    }
    *dev_ptr = p;
    *n_bytes = bytes;
    return DFL_OK;
}

dfl_status dfl_device_free(int32_t device, void* dev_ptr) {
    DFL_CHECK(use_device(device));
    if (dev_ptr) DFL_CUDA(cudaFree(dev_ptr));
    return DFL_OK;
}

dfl_status dfl_device_to_host(int32_t device, const void* dev_ptr, void* host, uint64_t n_bytes) {
    if (!dev_ptr || !host) return fail(DFL_ERR_BAD_ARG, "device_to_host: null argument");
    DFL_CHECK(use_device(device));
    DFL_CUDA(cudaMemcpy(host, dev_ptr, n_bytes, cudaMemcpyDeviceToHost));
    return DFL_OK;
}

}  // extern "C"
