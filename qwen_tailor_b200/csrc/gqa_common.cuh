// Shared pieces of the GQA decode attention kernels (gqa_decode.cu: warp-level MMA path for any page size and the work plan;
// gqa_decode_tc.cu: tcgen05 path for pages that hold a multiple of 64 keys).
#pragma once
#include <cuda.h>
#include "gdn_common.cuh"
#include "launchers.cuh"

namespace gdn {

constexpr int ATT_H = 8, ATT_KV = 2, ATT_D = 256, ATT_GQA = 4;
constexpr int TK = 64;                          // keys per tile
constexpr int ATT_THREADS = 256, KGROUPS = 4, KPW = TK / KGROUPS;      // 4 key groups of 16 keys x 2 dim halves
constexpr int ROWB = ATT_D * 2;                 // bytes per key row (512)
constexpr int TILE_BYTES = TK * ROWB;           // 32 KiB
constexpr int ATT_STAGES = 3;
constexpr int ATT_XCHG = 2 * KGROUPS * 2 * 32 * 16;                     // score exchange between the two warps of a key group, two buffers
constexpr int ATT_SMEM = 16 * ROWB + ATT_STAGES * 2 * TILE_BYTES + ATT_STAGES * TK * 8 + ATT_XCHG;     // Q (8 KiB) + stages x (K + V) + row offsets + exchange
constexpr int PART_STRIDE = 16 * ATT_D + 32;    // floats per (sequence, kv head, split): O[16][256] + (m, l)[16]


__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_k8(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(b0));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// byte offset of 16-byte chunk `c` of row `r` in a swizzled [rows][512 B] tile
__device__ __forceinline__ uint32_t swz(int r, int c) { return (uint32_t)(r * ROWB + ((c ^ (r & 7)) << 4)); }

// byte offset of 16-byte chunk `c` of key row `r` in a tile that TMA wrote as four [64 keys][64 dims] boxes with the 128-byte swizzle
__device__ __forceinline__ uint32_t swz_t(int r, int c) { return (uint32_t)((c >> 3) * 8192 + r * 128 + (((c & 7) ^ (r & 7)) << 4)); }

// ---- work plan in the workspace: ints meta[0] = total tiles, meta[1] = working blocks, then cum[P+1] (tile prefix sums per (sequence, kv head) pair),
//      base[P+1] (partial-slot prefix sums), first[P] (first block of each pair), count[P] (arrival counters, zeroed by the plan
//      kernel of every call); the fp32 partials follow ----
__host__ __device__ constexpr size_t meta_ints(int P) { return ((size_t)(4 + 4 * (P + 1)) + 63) / 64 * 64; }
__device__ __forceinline__ int* meta_cum(int* meta) { return meta + 4; }
__device__ __forceinline__ int* meta_base(int* meta, int P) { return meta + 4 + (P + 1); }
__device__ __forceinline__ int* meta_first(int* meta, int P) { return meta + 4 + 2 * (P + 1); }
__device__ __forceinline__ int* meta_count(int* meta, int P) { return meta + 4 + 3 * (P + 1); }     // partials written so far, per pair
// block that owns tile i when G blocks split N tiles as [c N / G, (c + 1) N / G)
__device__ __forceinline__ int block_of_tile(long long i, int G, long long N) { return (int)(((i + 1) * G - 1) / N); }


// the tcgen05 kernel (gqa_decode_tc.cu)
constexpr int TC_THREADS = 128;
constexpr int TC_MAX_PAIRS = 512;                                        // (sequence, KV head) pairs the kernel plans for in shared memory
constexpr int TC_Q_BYTES = 16384;                                      // Q operand: 4 slabs of 32 rows x 128 B (the 16 query rows, twice)
constexpr int TC_SMEM = TC_Q_BYTES + ATT_STAGES * 2 * TILE_BYTES;      // + three stages of K + V tiles
int launch_gqa_decode_tc(const AttnArgs& a, const CUtensorMap& tk, const CUtensorMap& tv, cudaStream_t stream);

}  // namespace gdn
