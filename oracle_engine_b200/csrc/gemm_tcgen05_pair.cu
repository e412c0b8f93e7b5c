// bf16 matrix product C (+)= A . W^T for many tokens (prompts) on pairs of SMs:
// tcgen05.mma.cta_group::2.  A cluster of two CTAs computes a 256 x n_tile output tile.  Each
// CTA loads its own 128 rows of the activations and HALF of the weight tile (n_tile/2 rows)
// by TMA into 128B-swizzled shared memory; one thread of the leader CTA issues the
// instructions, which read both CTAs' shared memory and write 128 rows of float32
// accumulators into each CTA's tensor memory.  Against the one-CTA kernel (gemm_tcgen05.cu)
// a k-block costs each SM 16 KB + n_tile * 64 bytes of operands instead of 16 KB +
// n_tile * 128 for the same tensor cycles; the path from the L2 into the SM is what limits
// the one-CTA kernel at these shapes.
//
// Roles per CTA (192 threads): warp 0 = TMA producer (its loads signal the LEADER's "full"
// barrier; no load uses cluster multicast), warp 1 = tensor-memory allocation (both CTAs, as a
// pair) and, in the leader, MMA issue; warps 2-5 = epilogue of the CTA's own 128 rows.  The
// leader frees a stage in both CTAs with one tcgen05.commit (multicast to the two CTAs'
// barriers) and announces a finished accumulator the same way; the epilogue warps of both CTAs
// arrive on the leader's "accumulator free" barrier.  Clusters are persistent and take output
// tiles round robin; two accumulators, so a tile's epilogue overlaps the next tile's products.
// Every wait on an mbarrier is bounded in time; a wait that runs out raises an error flag,
// every role leaves its loop (the partner's waits then run out too), copies in flight get a
// fixed time, both CTAs meet at the cluster barrier and free the tensor memory.
// Epilogues: bf16, float32, float32 accumulate (as reductions in the L2), SwiGLU on
// interleaved gate/up rows.  Takes the place of the reference's gemm_q for prompts
// (core/gguf_parser.cpp:913-997).
#include <cuda.h>
#include <cudaTypedefs.h>
#include "common.cuh"
#include <mutex>

namespace {

constexpr int BLOCK_M = 128;       // rows of a CTA's A tile; the pair's instruction has M = 256
constexpr int BLOCK_K = 64;        // bf16 per k-block = one 128-byte swizzled row
constexpr int UMMA_K = 16;
constexpr int A_TILE_BYTES = BLOCK_M * BLOCK_K * 2;      // 16 KB
constexpr int THREADS = 192;
constexpr int MAX_STAGES = 12;
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;   // 2 s

__device__ int g_error = 0;        // 0 = ok; else code of the wait that ran out

struct SharedCtl {
    uint64_t full[MAX_STAGES];     // used in the leader: both CTAs' loads of a stage have landed
    uint64_t empty[MAX_STAGES];    // in each CTA: the products have read the stage
    uint64_t tmem_full[2];         // in each CTA: an accumulator is complete
    uint64_t tmem_empty[2];        // used in the leader: both CTAs' epilogues have read it
    uint32_t tmem_base;
    int abort_flag;
};

struct PairArgs {
    void* C;
    long long ldc;
    int M, N, K;
    int n_tile;                    // columns of the pair's tile, multiple of 16, <= 256
    int acc_cols;                  // tensor-memory columns between the two accumulators (n_tile rounded up to 32)
    int stages;
    int out_kind;                  // 0 bf16 store, 1 float32 store, 2 float32 accumulate, 3 bf16 silu(gate)*up
    int tiles_m, tiles_n;          // tiles of 256 rows and of n_tile columns
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// The address, in the cluster's shared window, of the leader's copy of a shared variable.
__device__ __forceinline__ uint32_t in_leader(const void* p) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, 0;" : "=r"(r) : "r"(smem_u32(p)));
    return r;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive_in_leader(uint64_t* bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(in_leader(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, SharedCtl* ctl, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    for (uint32_t spin = 0;; spin++) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spin & 255u) == 255u) {
            if (*(volatile int*)&ctl->abort_flag) return false;
            if (global_ns() - t0 > WAIT_LIMIT_NS) {
                atomicExch(&ctl->abort_flag, 1);
                atomicCAS(&g_error, 0, code);
                return false;
            }
        }
    }
}
// A tile into this CTA's shared memory; completion is counted on the LEADER's barrier.
__device__ __forceinline__ void tma_load_pair(void* smem_dst, const CUtensorMap* map, uint32_t leader_bar, int c_inner, int c_outer) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"((uint64_t)map), "r"(leader_bar), "r"(c_inner), "r"(c_outer)
        : "memory");
}
// K-major tile, rows of 128 bytes, 128-byte swizzle, 8-row groups 1024 bytes apart, version 1 (sm_100).
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// kind::f16: D float32, A and B bf16, both K-major; m = 256 for the pair.
__device__ __forceinline__ uint32_t umma_idesc(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void umma_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrives on the barrier at this offset in BOTH CTAs when the products issued so far are done.
__device__ __forceinline__ void umma_commit_both(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// True in exactly one lane of a converged warp.  The warp stays converged around the
// instructions that lane issues, so their operands (descriptors, coordinates, barrier
// addresses) can stay in uniform registers.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}

__device__ __forceinline__ float silu_mul(float gate, float up) { return (gate / (1.f + expf(-gate))) * up; }
__device__ __forceinline__ void red_add(float* p, float v) { asm volatile("red.global.add.f32 [%0], %1;" ::"l"(p), "f"(v) : "memory"); }
__device__ __forceinline__ void red_add4(float* p, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// 16 consecutive columns (col0 ..) of output row `row`.  out_kind 3: the columns alternate gate, up.
__device__ __forceinline__ void emit16(const PairArgs& g, int row, int col0, const float (&v)[16]) {
    if (row >= g.M) return;
    const bool full = col0 + 16 <= g.N;
    if (g.out_kind == 3) {
        const long long base = (long long)row * g.ldc + (col0 >> 1);
        if (full && (base & 7) == 0) {
            uint32_t p[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                __nv_bfloat162 h = __floats2bfloat162_rn(silu_mul(v[4 * j], v[4 * j + 1]), silu_mul(v[4 * j + 2], v[4 * j + 3]));
                p[j] = *(uint32_t*)&h;
            }
            *(uint4*)((bf16*)g.C + base) = make_uint4(p[0], p[1], p[2], p[3]);
        } else {
#pragma unroll
            for (int j = 0; j < 8; j++)
                if (col0 + 2 * j + 1 < g.N) ((bf16*)g.C)[base + j] = __float2bfloat16_rn(silu_mul(v[2 * j], v[2 * j + 1]));
        }
        return;
    }
    const long long base = (long long)row * g.ldc + col0;
    if (full && g.out_kind == 0 && (base & 7) == 0) {
#pragma unroll
        for (int q = 0; q < 2; q++) {
            uint32_t p[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                __nv_bfloat162 h = __floats2bfloat162_rn(v[8 * q + 2 * j], v[8 * q + 2 * j + 1]);
                p[j] = *(uint32_t*)&h;
            }
            *(uint4*)((bf16*)g.C + base + 8 * q) = make_uint4(p[0], p[1], p[2], p[3]);
        }
    } else if (full && g.out_kind != 0 && (base & 3) == 0) {
        float4* dst = (float4*)((float*)g.C + base);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            if (g.out_kind == 2) red_add4((float*)(dst + j), v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            else dst[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        }
    } else {
#pragma unroll
        for (int j = 0; j < 16; j++) {
            if (col0 + j >= g.N) break;
            if (g.out_kind == 0) ((bf16*)g.C)[base + j] = __float2bfloat16_rn(v[j]);
            else if (g.out_kind == 1) ((float*)g.C)[base + j] = v[j];
            else red_add((float*)g.C + base + j, v[j]);
        }
    }
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const PairArgs g) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int b_half_rows = g.n_tile / 2;
    const int b_bytes = b_half_rows * BLOCK_K * 2;
    const int stage_bytes = A_TILE_BYTES + ((b_bytes + 1023) & ~1023);
    SharedCtl* ctl = (SharedCtl*)(smem + (size_t)g.stages * stage_bytes);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();
    const bool leader = rank == 0;
    const int cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
    const int n_work = g.tiles_m * g.tiles_n;
    const int n_kb = (g.K + BLOCK_K - 1) / BLOCK_K;
    uint32_t tmem_cols = 32;
    while ((int)tmem_cols < 2 * g.acc_cols) tmem_cols <<= 1;        // two accumulators

    if (threadIdx.x == 0) {
        for (int s = 0; s < g.stages; s++) { mbar_init(&ctl->full[s], 1); mbar_init(&ctl->empty[s], 1); }
        for (int b = 0; b < 2; b++) { mbar_init(&ctl->tmem_full[b], 1); mbar_init(&ctl->tmem_empty[b], 8); }
        ctl->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        // the two CTAs allocate the same columns of both tensor memories, as a pair
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl->tmem_base)), "r"(tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync();                                        // the partner's barriers exist before anything arrives on them
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *(volatile uint32_t*)&ctl->tmem_base;

    pdl_launch_dependents();
    if (warp == 0) {
        // ---------------- TMA producer (both CTAs) ----------------
        // The whole warp runs the loop and waits; one elected lane issues the copies.
        pdl_wait();                                        // the activations come from the kernel before
        int s = 0;                                         // the ring's next stage and its phase, over all tiles
        uint32_t phase = 0;
        bool ok = true;
        for (int w = cluster_id; w < n_work && ok; w += n_clusters) {
            const int tile_n = w / g.tiles_m, tile_m = w % g.tiles_m;
            const int a_row = tile_m * (2 * BLOCK_M) + (int)rank * BLOCK_M;
            const int b_row = tile_n * g.n_tile + (int)rank * b_half_rows;
            // a short loop per k-block (no division, addresses carried along): see gemm_tcgen05.cu
            for (int i = 0, col = 0; i < n_kb; i++, col += BLOCK_K) {
                if (!__all_sync(0xffffffffu, mbar_wait(&ctl->empty[s], phase ^ 1u, ctl, 1))) { ok = false; break; }
                if (elect_one()) {
                    uint8_t* a_dst = smem + (size_t)s * stage_bytes;
                    if (leader) mbar_expect_tx(&ctl->full[s], (uint32_t)(2 * (A_TILE_BYTES + b_bytes)));
                    const uint32_t bar = in_leader(&ctl->full[s]);
                    tma_load_pair(a_dst, &map_a, bar, col, a_row);
                    tma_load_pair(a_dst + A_TILE_BYTES, &map_b, bar, col, b_row);
                }
                __syncwarp();
                if (++s == g.stages) { s = 0; phase ^= 1u; }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issue (leader only) ----------------
        // The whole warp runs the loop and waits; one elected lane issues the instructions.
        if (leader) {
            const uint32_t idesc = umma_idesc(2 * BLOCK_M, g.n_tile);
            int lt = 0;
            int s = 0;
            uint32_t phase = 0;
            // descriptors differ between stages and 16-deep steps only in their address field (bytes / 16)
            const uint64_t desc0 = umma_desc(smem_u32(smem));
            const uint64_t stage_step = (uint64_t)(stage_bytes >> 4), b_step = (uint64_t)(A_TILE_BYTES >> 4);
            bool ok = true;
            for (int w = cluster_id; w < n_work && ok; w += n_clusters, lt++) {
                const int buf = lt & 1;
                // both CTAs' epilogues have read this accumulator (two tiles ago)
                if (!__all_sync(0xffffffffu, mbar_wait(&ctl->tmem_empty[buf], ((uint32_t)(lt >> 1) & 1u) ^ 1u, ctl, 4))) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tmem_d = tmem_base + (uint32_t)(buf * g.acc_cols);
                for (int i = 0; i < n_kb; i++) {
                    if (!__all_sync(0xffffffffu, mbar_wait(&ctl->full[s], phase, ctl, 2))) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    if (elect_one()) {
                        const uint64_t a_desc = desc0 + (uint64_t)s * stage_step, b_desc = a_desc + b_step;
                        umma_pair(tmem_d, a_desc, b_desc, idesc, i > 0 ? 1u : 0u);
#pragma unroll
                        for (int k = 1; k < BLOCK_K / UMMA_K; k++)
                            umma_pair(tmem_d, a_desc + (uint64_t)(k * UMMA_K * 2 >> 4), b_desc + (uint64_t)(k * UMMA_K * 2 >> 4), idesc, 1u);
                        umma_commit_both(&ctl->empty[s]);   // frees the stage in both CTAs
                    }
                    __syncwarp();
                    if (++s == g.stages) { s = 0; phase ^= 1u; }
                }
                if (ok) {
                    if (elect_one()) umma_commit_both(&ctl->tmem_full[buf]);
                    __syncwarp();
                }
            }
        }
    } else {
        // ---------------- epilogue: warps 2..5 of both CTAs, the CTA's own 128 rows ----------------
        const int quarter = warp & 3;
        const int row_in_cta = quarter * 32 + lane;
        int lt = 0;
        bool first = true;
        for (int w = cluster_id; w < n_work; w += n_clusters, lt++) {
            const int tile_n = w / g.tiles_m, tile_m = w % g.tiles_m;
            const int row = tile_m * (2 * BLOCK_M) + (int)rank * BLOCK_M + row_in_cta;
            const int buf = lt & 1;
            if (!mbar_wait(&ctl->tmem_full[buf], (uint32_t)(lt >> 1) & 1u, ctl, 3)) break;
            if (first) { pdl_wait(); first = false; }     // before the first access to C
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * g.acc_cols);
            for (int c0 = 0; c0 < g.n_tile; c0 += 32) {    // n_tile is a multiple of 16: the last group may be half
                uint32_t r[2][16];
                const bool two = c0 + 16 < g.n_tile;
                tmem_ld16(taddr + (uint32_t)c0, r[0]);
                if (two) tmem_ld16(taddr + (uint32_t)(c0 + 16), r[1]);
                tmem_ld_wait();
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    if (h == 1 && !two) break;
                    float v[16];
#pragma unroll
                    for (int j = 0; j < 16; j++) v[j] = __uint_as_float(r[h][j]);
                    emit16(g, row, tile_n * g.n_tile + c0 + 16 * h, v);
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_in_leader(&ctl->tmem_empty[buf]);
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }

    __syncthreads();
    if (*(volatile int*)&ctl->abort_flag) {
        const unsigned long long t0 = global_ns();
        while (global_ns() - t0 < 2000000ull) __nanosleep(1000);
        __syncthreads();
    }
    cluster_sync();                                        // neither CTA leaves while the other may still use its memories
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
    }
}

PFN_cuTensorMapEncodeTiled_v12000 g_encode = nullptr;
std::mutex g_mutex;

int get_encode() {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (g_encode) return 0;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || fn == nullptr) return e != cudaSuccess ? (int)e : 999;
    g_encode = (PFN_cuTensorMapEncodeTiled_v12000)fn;
    return 0;
}

int make_map(CUtensorMap* map, const void* ptr, long long rows, long long K, long long ld, int box_rows) {
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)BLOCK_K, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : 1000 + (int)r;
}

int g_clusters = -1;               // clusters of two CTAs that the device runs at once

}  // namespace

extern "C" {

// 1 if the pair kernel takes these operands (more than 128 tokens; TMA needs 16-byte aligned rows).
int oe_gemm_pair_supported(const void* A, const void* W, int M, int N, int K, long long lda) {
    if (M <= 128 || N < 32 || K <= 0) return 0;
    if ((K % 8) || (lda % 8)) return 0;
    if (((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return 0;
    return 1;
}

// C[M,N] (+)= A[M,K] . W[N,K]^T ; out_kind: 0 bf16, 1 float32, 2 float32 accumulate,
// 3: W's rows alternate gate/up and C[M,N/2] = silu(gate) * up as bf16 (ldc counts C's elements).
// max_tile: 0, or an upper limit for the tile's columns (for tests).
int oe_gemm_pair_bf16(void* C, const bf16* A, const bf16* W, int M, int N, int K, long long lda, long long ldc,
                      int out_kind, int max_tile, cudaStream_t st) {
    if (!oe_gemm_pair_supported(A, W, M, N, K, lda)) return OE_ERR_UNSUPPORTED;
    if (out_kind < 0 || out_kind > 3 || (out_kind == 3 && (N & 1))) return OE_ERR_UNSUPPORTED;
    int rc = get_encode();
    if (rc) return rc;
    const size_t smem_max = 227 * 1024;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_max);
        if (e != cudaSuccess) return (int)e;
        attr_set = true;
    }
    if (g_clusters < 0) {
        cudaLaunchConfig_t probe = {};
        probe.gridDim = dim3(2); probe.blockDim = dim3(THREADS); probe.dynamicSmemBytes = smem_max;
        int n = 0;
        cudaError_t e = cudaOccupancyMaxActiveClusters(&n, gemm_pair_kernel, &probe);
        if (e != cudaSuccess) return (int)e;
        if (n < 1) return OE_ERR_UNSUPPORTED;
        g_clusters = n;
    }
    PairArgs g;
    g.C = C; g.ldc = ldc; g.M = M; g.N = N; g.K = K; g.out_kind = out_kind;
    g.tiles_m = (M + 2 * BLOCK_M - 1) / (2 * BLOCK_M);
    // The tile width (a multiple of 16) with the shortest rounds of clusters at the measured time of a
    // pair's k-block: 230, 249, 284, 310 and 365 ns from 128, 160, 192, 224 and 256 columns on, and a
    // width between two of these costs what the one below it costs (4096^3 with every width forced,
    // the roles as converged warps).  So 176 columns are the cheapest per column after 224..256, and
    // 8192 -> 3072 at 2,048 tokens takes 18 x 8 tiles of 176 (1.95 rounds of 74 clusters) rather than
    // 16 x 8 of 192 (1.73 rounds).
    int limit = 256;
    if (max_tile >= 32 && max_tile < limit) limit = max_tile / 16 * 16;
    long long best = -1;
    g.n_tile = limit;
    for (int nt = limit; nt >= 128 && nt >= 32; nt -= 16) {
        const long long tiles = (long long)g.tiles_m * ((N + nt - 1) / nt);
        static const int kb_ns[9] = {230, 230, 230, 230, 230, 249, 284, 310, 365};
        const long long cost = ((tiles + g_clusters - 1) / g_clusters) * kb_ns[nt / 32];
        if (best < 0 || cost < best) { best = cost; g.n_tile = nt; }
    }
    if (max_tile <= -32 && max_tile >= -256 && max_tile % 16 == 0) g.n_tile = -max_tile;     // measurements: this width
    if (N < g.n_tile) g.n_tile = (N + 15) / 16 * 16;
    g.acc_cols = (g.n_tile + 31) / 32 * 32;
    g.tiles_n = (N + g.n_tile - 1) / g.n_tile;
    const long long n_work = (long long)g.tiles_m * g.tiles_n;
    if (n_work > 2147483647LL) return OE_ERR_UNSUPPORTED;
    CUtensorMap map_a, map_b;
    if ((rc = make_map(&map_a, A, M, K, lda, BLOCK_M))) return rc;
    if ((rc = make_map(&map_b, W, N, K, K, g.n_tile / 2))) return rc;
    const int n_kb = (K + BLOCK_K - 1) / BLOCK_K;
    const int b_bytes = (g.n_tile / 2) * BLOCK_K * 2;
    const int stage_bytes = A_TILE_BYTES + ((b_bytes + 1023) & ~1023);
    int stages = (200 * 1024) / stage_bytes;
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    if (stages > n_kb) stages = n_kb < 2 ? 2 : n_kb;
    g.stages = stages;
    const size_t smem = (size_t)stages * stage_bytes + sizeof(SharedCtl) + 1024;
    const int clusters = (int)(n_work < g_clusters ? n_work : g_clusters);
    return oe_launch(gemm_pair_kernel, dim3(2 * clusters), dim3(THREADS), smem, st, map_a, map_b, g);
}

// Reads and clears the device-side error flag (0 = no wait ran out).
int oe_gemm_pair_error() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_error, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) cudaMemcpyToSymbol(g_error, &zero, sizeof(int));
    return v;
}

}  // extern "C"
