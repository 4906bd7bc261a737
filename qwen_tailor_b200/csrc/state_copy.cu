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

// Row scatter of the speculative mode's hidden-state history (the reference's `hrec` kernel, qwen35/batch.py:375-399):
//     hist[slots[b], pos[b], :] = rows[b, :]        hist [n_slots, Lh, H] bf16, rows [B, H] bf16
// The indices live on the device; a row whose slot or position is out of range is skipped and reported through the status word.
__global__ void hrec_kernel(__nv_bfloat16* __restrict__ hist, const __nv_bfloat16* __restrict__ rows, const int* __restrict__ slots,
                            const int* __restrict__ pos, int n_slots, int Lh, int H, int* status) {
    const int b = blockIdx.y;
    const int s = slots[b], p = pos[b];
    if (s < 0 || s >= n_slots || p < 0 || p >= Lh) { if (threadIdx.x == 0 && blockIdx.x == 0) atomicExch(status, 1); return; }
    __nv_bfloat16* d = hist + ((size_t)s * Lh + p) * H;
    const __nv_bfloat16* r = rows + (size_t)b * H;
    const bool vec = (H % 8 == 0) && (reinterpret_cast<uintptr_t>(d) % 16 == 0) && (reinterpret_cast<uintptr_t>(r) % 16 == 0);
    if (vec) {
        for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < H / 8; i += gridDim.x * blockDim.x)
            reinterpret_cast<uint4*>(d)[i] = reinterpret_cast<const uint4*>(r)[i];
    } else {
        for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < H; i += gridDim.x * blockDim.x) d[i] = r[i];
    }
}

int launch_hrec(void* hist, const void* rows, const int* slots, const int* pos, int B, int n_slots, int Lh, int H, int* status, cudaStream_t st) {
    if (B <= 0 || H <= 0) return GDN_OK;
    if (B > 65535) { set_error("hrec: B = %d exceeds 65535", B); return GDN_E_SHAPE; }
    hrec_kernel<<<dim3(1, B), 128, 0, st>>>(static_cast<__nv_bfloat16*>(hist), static_cast<const __nv_bfloat16*>(rows), slots, pos, n_slots, Lh, H, status);
    return check_launch("hrec");
}

}  // namespace gdn
