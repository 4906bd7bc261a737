// Strided in-place copies for state admission, snapshot moves and prefix-cache checkpoints.
//
// Replaces the reference's `blit` kernel (qwen35/batch.py:349-372):
//     dst.flat[d0 + y*dstride + i] = src.flat[s0 + y*sstride + i]   for i < n, y < ny
// Offsets and strides are in elements of `elem_size` bytes (2 = bf16, 4 = fp32).  Rows are copied with 16-byte accesses when
// every address involved is 16-byte aligned, element by element otherwise.
#include "gdn_common.cuh"

namespace gdn {

template <typename T>
__global__ void state_copy_kernel(T* __restrict__ dst, const T* __restrict__ src, long long n, long long dstride, long long sstride) {
    const long long y = blockIdx.y;
    T* d = dst + y * dstride;
    const T* s = src + y * sstride;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) d[i] = s[i];
}

template <typename T>
static int run(void* dst, const void* src, long long n, long long d0, long long s0, int ny, long long dstride, long long sstride, cudaStream_t st) {
    long long blocks = (n + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    state_copy_kernel<T><<<dim3((unsigned)blocks, ny), 256, 0, st>>>(static_cast<T*>(dst) + d0, static_cast<const T*>(src) + s0, n, dstride, sstride);
    return check_launch("state_copy");
}

int launch_state_copy(void* dst, const void* src, int elem_size, long long n, long long d0, long long s0, int ny, long long dstride,
                      long long sstride, cudaStream_t st) {
    if (n <= 0 || ny <= 0) return GDN_OK;
    if (elem_size != 2 && elem_size != 4) { set_error("state_copy: elem_size must be 2 or 4, got %d", elem_size); return GDN_E_DTYPE; }
    if (ny > 65535) { set_error("state_copy: ny = %d exceeds 65535", ny); return GDN_E_SHAPE; }
    const long long per16 = 16 / elem_size;
    const bool vec = (n % per16 == 0) && (d0 % per16 == 0) && (s0 % per16 == 0) && (dstride % per16 == 0) && (sstride % per16 == 0) &&
                     (reinterpret_cast<uintptr_t>(dst) % 16 == 0) && (reinterpret_cast<uintptr_t>(src) % 16 == 0);
    if (vec) return run<uint4>(dst, src, n / per16, d0 / per16, s0 / per16, ny, dstride / per16, sstride / per16, st);
    if (elem_size == 4) return run<uint32_t>(dst, src, n, d0, s0, ny, dstride, sstride, st);
    return run<uint16_t>(dst, src, n, d0, s0, ny, dstride, sstride, st);
}

}  // namespace gdn
