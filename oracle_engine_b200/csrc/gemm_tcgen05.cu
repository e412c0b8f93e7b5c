// bf16 matrix product C (+)= A . W^T on the 5th-generation tensor cores (sm_100a):
// TMA (cp.async.bulk.tensor) stages K-major operand tiles in 128B-swizzled shared memory,
// one thread issues tcgen05.mma with float32 accumulators in tensor memory, four warps
// read the accumulators back with tcgen05.ld and store.
//
// Both operands are [rows, K] row-major (activations [tokens, K], weights [out, K]), which
// is the K-major form the instruction takes without a transpose.  The kernel works on an
// "A" operand whose tile is 128 rows (the M of the instruction) and a "B" operand whose
// tile is n_tile rows (16..256, the N of the instruction):
//   * many tokens (prompts): A = activations, B = weights, n_tile = 128 or 256;
//   * few tokens (decode):   A = weights, B = activations ("swap"), n_tile = tokens rounded
//     up to 16, the output tile is stored transposed, and K is split over several CTAs so
//     that all SMs stream weights.  The partial sums of a split go through a float32
//     workspace and the CTA that finishes last adds them in split order (deterministic).
// Roles per CTA (192 threads): warp 0 = TMA producer, warp 1 = TMEM allocation and MMA
// issue, warps 2-5 = epilogue.  Every wait on an mbarrier is bounded in time; a wait that
// runs out sets an error flag, lets every role leave its loop, waits a fixed time for
// copies in flight, frees the tensor memory and returns.  The host reads the flag with
// oe_gemm_tc_error().
// Takes the place of the reference's gemm_q / gemv_q (core/gguf_parser.cpp:868-997).
#include <cuda.h>
#include <cudaTypedefs.h>
#include "common.cuh"
#include <mutex>
#include <unordered_map>

namespace {

constexpr int BLOCK_M = 128;       // rows of the A tile = UMMA M
constexpr int BLOCK_K = 64;        // bf16 per swizzle atom = one 128-byte swizzled row; a k-block is 1 or 2 atoms
constexpr int UMMA_K = 16;
constexpr int A_TILE_BYTES = BLOCK_M * BLOCK_K * 2;      // 16 KB
constexpr int THREADS = 192;
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;   // 2 s: the default limit of every wait (GemmArgs::wait_ns)

__device__ int g_error = 0;        // 0 = ok; else code of the wait that ran out

struct SharedCtl {
    uint64_t full[12];
    uint64_t empty[12];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    unsigned long long wait_ns;      // limit of every wait on an mbarrier
    uint32_t tmem_base;
    int abort_flag;
    int is_last;
    int epi_ok;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// True in exactly one lane of a converged warp.  The TMA and MMA roles are run by whole warps
// that stay converged, and this lane issues: inside `if (lane == 0)` every operand of every
// copy and instruction (descriptors, coordinates, barrier addresses) went through that one
// lane's registers, which cost more per k-block than the tensor cores needed.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// The address of this CTA's shared-memory address `a` in the CTA of rank `rank` of the cluster.
__device__ __forceinline__ uint32_t peer_smem(uint32_t a, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(rank));
    return r;
}
__device__ __forceinline__ float4 ld_cluster_f4(uint32_t a) {
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(a) : "memory");
    return v;
}
// Every thread of every CTA of the cluster calls it (threads that have left count as arrived).
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
}

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
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
// Waits for the phase with `parity` to complete; gives up after the limit (ctl->wait_ns) or
// when another role has given up, and then returns false.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, SharedCtl* ctl, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    for (uint32_t spin = 0;; spin++) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spin & 255u) == 255u) {
            if (*(volatile int*)&ctl->abort_flag) return false;
            if (global_ns() - t0 > ctl->wait_ns) {
                atomicExch(&ctl->abort_flag, 1);
                atomicCAS(&g_error, 0, code);
                return false;
            }
        }
    }
}

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c_inner, int c_outer) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"((uint64_t)map), "r"(smem_u32(bar)), "r"(c_inner), "r"(c_outer)
        : "memory");
}

// Shared-memory matrix descriptor: K-major tile, rows of 128 bytes, 128-byte swizzle,
// 8-row groups 1024 bytes apart (stride byte offset), descriptor version 1 (sm_100).
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;                    // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;          // stride byte offset
    d |= (uint64_t)1 << 46;                    // version
    d |= (uint64_t)2 << 61;                    // SWIZZLE_128B
    return d;
}

// Instruction descriptor of tcgen05.mma.kind::f16: D float32, A and B bf16, both K-major.
__device__ __forceinline__ uint32_t umma_idesc(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

struct GemmArgs {
    void* C;
    long long ldc;
    int rows_a, rows_b, K;      // valid rows of the A (128-row) and B (n_tile-row) operands
    int n_tile;                 // rows of the B tile, multiple of 16, <= 256
    int atoms;                  // 64-deep swizzle atoms per k-block and pipeline stage (1 or 2)
    int n_kb_total, kb_per;     // k-blocks of the whole K, and of one split (worked out on the host: no division per thread)
    int stages;
    int swap;                   // 1: C[b_row, a_row] (A = weights); 0: C[a_row, b_row] (A = activations)
    int out_kind;               // 0 bf16 store, 1 float32 store, 2 float32 accumulate, 3 bf16 silu(gate)*up
    int splits;
    int tiles_a, tiles_b;       // output tiles along the A and the B operand
    int streamk;                // 1: the CTAs share the k-blocks of the first sk_tiles tiles equally (see ItemIter)
    int sk_tiles;
    int cluster;                // > 1: the K splits of a tile are the CTAs of one cluster, which add up through shared memory
    float* workspace;           // [splits][tiles_a][tiles_b][n_tile][128] float32 when splits > 1
    int* counters;              // [tiles_a * tiles_b], zero between launches
    unsigned long long wait_ns; // after this long a wait on an mbarrier gives up (error flag, the kernel returns)
    const uint8_t* pf_ptr;      // the weights of the product after this one: their first pf_bytes are asked into the L2
    long long pf_bytes;         // by this kernel's TMA role once its own loads are out (0: none)
    int withhold_release;       // tests of that path: the epilogue never hands an accumulator back, so that the
                                // MMA role's wait for one runs out (0 in every other use)
};

// Accumulation into C goes out as reductions that the L2 performs (no load on the SM's side, so
// the epilogue does not wait for memory).  Every element of C gets exactly one addition per
// product, so the result does not depend on the order in which the reductions arrive.
__device__ __forceinline__ void red_add(float* p, float v) {
    asm volatile("red.global.add.f32 [%0], %1;" ::"l"(p), "f"(v) : "memory");
}
__device__ __forceinline__ void red_add4(float* p, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
__device__ __forceinline__ void store_out(const GemmArgs& g, long long idx, float v) {
    if (g.out_kind == 0) ((bf16*)g.C)[idx] = __float2bfloat16_rn(v);
    else if (g.out_kind == 1) ((float*)g.C)[idx] = v;
    else red_add((float*)g.C + idx, v);
}

__device__ __forceinline__ float silu_mul(float gate, float up) { return (gate / (1.f + expf(-gate))) * up; }

// Stores NC consecutive B-rows (b_row0 ..) of A-row `a_row` of the output tile.  Called by all
// 32 lanes of a warp together (out_kind 3 exchanges values between neighbouring lanes).
// out_kind 3: rows of the weight matrix alternate gate, up (g0, u0, g1, u1, ...); the output
// is silu(gate) * up as bf16, half as many features.
template <int NC>
__device__ __forceinline__ void emit(const GemmArgs& g, int a_row, int b_row0, const float (&v)[NC]) {
    const bool a_ok = a_row < g.rows_a;
    if (g.swap) {
        if (g.out_kind == 3) {
#pragma unroll
            for (int j = 0; j < NC; j++) {
                const float other = __shfl_xor_sync(0xffffffffu, v[j], 1);
                const int b_row = b_row0 + j;
                if (a_ok && !(a_row & 1) && b_row < g.rows_b)
                    ((bf16*)g.C)[(long long)b_row * g.ldc + (a_row >> 1)] = __float2bfloat16_rn(silu_mul(v[j], other));
            }
        } else if (a_ok) {
#pragma unroll
            for (int j = 0; j < NC; j++) {
                const int b_row = b_row0 + j;
                if (b_row < g.rows_b) store_out(g, (long long)b_row * g.ldc + a_row, v[j]);
            }
        }
        return;
    }
    if (!a_ok) return;
    const bool full = b_row0 + NC <= g.rows_b;
    if (g.out_kind == 3) {
        const long long base = (long long)a_row * g.ldc + (b_row0 >> 1);
        if (full && NC == 16 && (base & 7) == 0) {
            uint32_t p[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                __nv_bfloat162 h = __floats2bfloat162_rn(silu_mul(v[4 * j], v[4 * j + 1]), silu_mul(v[4 * j + 2], v[4 * j + 3]));
                p[j] = *(uint32_t*)&h;
            }
            *(uint4*)((bf16*)g.C + base) = make_uint4(p[0], p[1], p[2], p[3]);
        } else {
#pragma unroll
            for (int j = 0; j < NC / 2; j++)
                if (b_row0 + 2 * j + 1 < g.rows_b) ((bf16*)g.C)[base + j] = __float2bfloat16_rn(silu_mul(v[2 * j], v[2 * j + 1]));
        }
        return;
    }
    const long long base = (long long)a_row * g.ldc + b_row0;
    if (full && g.out_kind == 0 && (base & 7) == 0) {
#pragma unroll
        for (int q = 0; q < NC / 8; q++) {
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
        for (int j = 0; j < NC / 4; j++) {
            if (g.out_kind == 2) red_add4((float*)(dst + j), v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            else dst[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        }
    } else {
#pragma unroll
        for (int j = 0; j < NC; j++)
            if (b_row0 + j < g.rows_b) store_out(g, base + j, v[j]);
    }
}

// The work items of a CTA.
// Tile mode: output tiles (times K splits), taken round robin by the resident CTAs; A-tiles vary
// fastest, so CTAs that run together share the B tile in L2.
// Stream-K mode (many tokens, a tile count that does not fill the last round of CTAs): an
// instruction of any width up to 256 costs about the same, so a k-block of a 128 x 256 tile is
// the unit of work.  The k-blocks of the first sk_tiles tiles, in tile order, are cut into
// gridDim.x equal runs: a CTA's run is the tail of one tile, whole tiles, and the head of
// another.  The other tiles (a multiple of gridDim.x) follow round robin, whole, so every SM
// multiplies the same number of k-blocks whatever the shape, and the sums of the shared
// tiles are added up by the epilogue warps while the whole tiles are multiplied.  The pieces
// of a shared tile go through the workspace (slot 2 c for CTA c's first item, 2 c + 1 for
// its last), and the CTA that arrives last on the tile's counter adds them in k order and
// stores: no CTA waits for another.
struct Item {
    int tile_a, tile_b, kb0, n_kb;
    int n_parts, my_part;       // pieces of this tile and which one this is (1, 0: the whole tile)
    int split;                  // tile mode: the K split
    int c_first;                // stream-K: the CTA that has the tile's first k-block
};
struct ItemIter {
    int streamk, cluster, tiles_a, tiles_b, splits, n_kb_total, kb_per;
    int w, step, n_work;                        // tile mode
    long long u, u0, u1, T;                     // stream-K: this CTA's run of k-block units and the total
    long long dp, n_tiles;                      // stream-K: the next whole tile of this CTA
    int G;
    __device__ long long start_of(int c) const { return T * c / G; }
    __device__ int cta_of(long long unit) const {
        int c = (int)(unit * G / T);
        while (c + 1 < G && start_of(c + 1) <= unit) c++;
        while (c > 0 && start_of(c) > unit) c--;
        return c;
    }
    __device__ bool next(Item& it) {
        if (streamk) {
            if (u >= u1) {
                if (dp >= n_tiles) return false;
                it.tile_b = (int)(dp / tiles_a); it.tile_a = (int)(dp % tiles_a);
                it.kb0 = 0; it.n_kb = n_kb_total; it.split = 0;
                it.n_parts = 1; it.my_part = 0; it.c_first = (int)blockIdx.x;
                dp += G;
                return true;
            }
            const long long tile = u / n_kb_total;
            it.kb0 = (int)(u % n_kb_total);
            long long n = u1 - u;
            if (n > n_kb_total - it.kb0) n = n_kb_total - it.kb0;
            it.n_kb = (int)n;
            it.tile_b = (int)(tile / tiles_a); it.tile_a = (int)(tile % tiles_a);
            it.split = 0;
            if (it.n_kb == n_kb_total) { it.n_parts = 1; it.my_part = 0; it.c_first = (int)blockIdx.x; }
            else {
                it.c_first = cta_of(tile * n_kb_total);
                it.n_parts = cta_of((tile + 1) * n_kb_total - 1) - it.c_first + 1;
                it.my_part = (int)blockIdx.x - it.c_first;
            }
            u += n;
            return true;
        }
        if (w >= n_work) return false;
        // in a cluster the splits of a tile are neighbours (the cluster's ranks)
        const int rem = cluster > 1 ? w / splits : w % (tiles_a * tiles_b);
        it.split = cluster > 1 ? w % splits : w / (tiles_a * tiles_b); it.tile_b = rem / tiles_a; it.tile_a = rem % tiles_a;
        it.kb0 = it.split * kb_per;
        it.n_kb = min(n_kb_total, it.kb0 + kb_per) - it.kb0;
        it.n_parts = splits; it.my_part = it.split; it.c_first = 0;
        w += step;
        return true;
    }
};
__device__ __forceinline__ ItemIter make_iter(const GemmArgs& g) {
    ItemIter t;
    t.streamk = g.streamk; t.cluster = g.cluster; t.tiles_a = g.tiles_a; t.tiles_b = g.tiles_b; t.splits = g.splits;
    t.n_kb_total = g.n_kb_total;
    t.kb_per = g.kb_per;
    t.w = blockIdx.x; t.step = gridDim.x; t.n_work = g.tiles_a * g.tiles_b * g.splits;
    t.G = gridDim.x;
    t.T = 0; t.n_tiles = 0; t.dp = 0; t.u0 = t.u1 = t.u = 0;
    if (g.streamk) {           // 64-bit divisions: only where the schedule needs them
        t.T = (long long)g.sk_tiles * t.n_kb_total;
        t.n_tiles = (long long)g.tiles_a * g.tiles_b; t.dp = (long long)g.sk_tiles + blockIdx.x;
        t.u0 = t.start_of(blockIdx.x); t.u1 = t.start_of(blockIdx.x + 1); t.u = t.u0;
    }
    return t;
}
// Where piece p of the item's tile lies in the workspace (floats), for row 0 and column 0.
__device__ __forceinline__ size_t part_base(const GemmArgs& g, const ItemIter& t, const Item& it, int p) {
    const size_t tile_floats = (size_t)g.n_tile * BLOCK_M;
    if (g.streamk) {
        const int c = it.c_first + p;
        const long long tile = (long long)it.tile_b * g.tiles_a + it.tile_a;
        const int slot = 2 * c + ((t.start_of(c) / t.n_kb_total == tile) ? 0 : 1);
        return (size_t)slot * tile_floats;
    }
    return ((size_t)p * g.tiles_a * g.tiles_b + (size_t)it.tile_a * g.tiles_b + it.tile_b) * tile_floats;
}

__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const GemmArgs g) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // tiles first (1024-byte aligned for the 128-byte swizzle), control block after them
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    // a stage: the A tile's atoms (128 rows x 128 bytes each), then the B tile's
    const int b_tile_bytes = g.n_tile * BLOCK_K * 2;
    const int b_atom_bytes = (b_tile_bytes + 1023) & ~1023;
    const int stage_bytes = g.atoms * (A_TILE_BYTES + b_atom_bytes);
    const int b_off = g.atoms * A_TILE_BYTES;
    const int kb_elems = BLOCK_K * g.atoms;
    const uint32_t stage_tx = (uint32_t)(g.atoms * (A_TILE_BYTES + b_tile_bytes));
    SharedCtl* ctl = (SharedCtl*)(smem + (size_t)g.stages * stage_bytes);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_b = g.tiles_b;
    uint32_t tmem_cols = 32;
    while ((int)tmem_cols < 2 * g.n_tile) tmem_cols <<= 1;          // two accumulators

    if (threadIdx.x == 32) {    // the copies' descriptors are on their way while the barriers are set up
        asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)&map_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)&map_b) : "memory");
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < g.stages; s++) { mbar_init(&ctl->full[s], 1); mbar_init(&ctl->empty[s], 1); }
        for (int b = 0; b < 2; b++) { mbar_init(&ctl->tmem_full[b], 1); mbar_init(&ctl->tmem_empty[b], 4); }
        ctl->abort_flag = 0;
        ctl->wait_ns = g.wait_ns;
        ctl->is_last = 0;
        ctl->epi_ok = 1;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl->tmem_base)), "r"(tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *(volatile uint32_t*)&ctl->tmem_base;

    int cl_tile_a = 0, cl_tile_b = 0;             // cluster mode: the tile of this CTA's work item
    pdl_launch_dependents();
    if (warp == 0) {
        // ---------------- TMA producer ----------------
        // The weight operand (A when swapped, else B) does not depend on earlier kernels:
        // the first stages' weight tiles are requested before pdl_wait(), the activation
        // tiles after it.
        {
            int s = 0;                                          // the ring's next stage, over all work items
            uint32_t phase = 0;                                 // and how often the ring has wrapped (mod 2)
            bool waited = false, ok = true;
            ItemIter iter = make_iter(g);
            Item item;
            while (ok && iter.next(item)) {
                const int tile_b = item.tile_b, tile_a = item.tile_a, kb0 = item.kb0, n_kb = item.n_kb;
                int i = 0;
                if (!waited) {
                    const int first = min(n_kb, g.stages);
                    if (elect_one()) {
                        for (int j = 0; j < first; j++) {
                            uint8_t* a_dst = smem + (size_t)j * stage_bytes;
                            mbar_expect_tx(&ctl->full[j], stage_tx);
                            for (int h = 0; h < g.atoms; h++) {
                                if (g.swap) tma_load_2d(a_dst + h * A_TILE_BYTES, &map_a, &ctl->full[j], (kb0 + j) * kb_elems + h * BLOCK_K, tile_a * BLOCK_M);
                                else tma_load_2d(a_dst + b_off + h * b_atom_bytes, &map_b, &ctl->full[j], (kb0 + j) * kb_elems + h * BLOCK_K, tile_b * g.n_tile);
                            }
                        }
                    }
                    __syncwarp();
                    pdl_wait();
                    waited = true;
                    if (elect_one()) {
                        for (int j = 0; j < first; j++) {
                            uint8_t* a_dst = smem + (size_t)j * stage_bytes;
                            for (int h = 0; h < g.atoms; h++) {
                                if (g.swap) tma_load_2d(a_dst + b_off + h * b_atom_bytes, &map_b, &ctl->full[j], (kb0 + j) * kb_elems + h * BLOCK_K, tile_b * g.n_tile);
                                else tma_load_2d(a_dst + h * A_TILE_BYTES, &map_a, &ctl->full[j], (kb0 + j) * kb_elems + h * BLOCK_K, tile_a * BLOCK_M);
                            }
                        }
                    }
                    __syncwarp();
                    i = first;
                    s = first == g.stages ? 0 : first;          // the ring's next stage and its phase
                    phase = first == g.stages ? 1u : 0u;
                }
                // The loop of one k-block is short on purpose (no division, addresses carried along):
                // the warp that runs it is one of two whose rate bounds what a CTA streams.
                const int row_a = tile_a * BLOCK_M, row_b = tile_b * g.n_tile;
                int col = (kb0 + i) * kb_elems;
                for (; i < n_kb; i++, col += kb_elems) {
                    if (!__all_sync(0xffffffffu, mbar_wait(&ctl->empty[s], phase ^ 1u, ctl, 1))) { ok = false; break; }
                    if (elect_one()) {
                        uint8_t* a_dst = smem + (size_t)s * stage_bytes;
                        mbar_expect_tx(&ctl->full[s], stage_tx);
                        tma_load_2d(a_dst, &map_a, &ctl->full[s], col, row_a);
                        tma_load_2d(a_dst + b_off, &map_b, &ctl->full[s], col, row_b);
                        if (g.atoms == 2) {
                            tma_load_2d(a_dst + A_TILE_BYTES, &map_a, &ctl->full[s], col + BLOCK_K, row_a);
                            tma_load_2d(a_dst + b_off + b_atom_bytes, &map_b, &ctl->full[s], col + BLOCK_K, row_b);
                        }
                    }
                    __syncwarp();
                    if (++s == g.stages) { s = 0; phase ^= 1u; }
                }
            }
            // This CTA's own loads are on their way.  While its last MMAs, its epilogue and the next kernel's
            // set-up run, the memory would idle: the first bytes of the next product's weights go to the L2.
            if (g.pf_bytes > 0 && elect_one()) {
                const long long per = ((g.pf_bytes / gridDim.x) + 127) & ~127ll;
                const long long begin = (long long)blockIdx.x * per;
                const long long n = min(per, g.pf_bytes - begin);
                for (long long off = 0; off < n; off += 32768) {
                    const uint32_t sz = (uint32_t)min(32768ll, n - off) & ~15u;
                    if (sz) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(g.pf_ptr + begin + off), "r"(sz) : "memory");
                }
            }
            __syncwarp();
        }
    } else if (warp == 1) {
        // ---------------- MMA issue ----------------
        {
            const uint32_t idesc = umma_idesc(BLOCK_M, g.n_tile);
            int lt = 0;
            int s = 0;                                          // the ring's next stage and its phase, over all work items
            uint32_t phase = 0;
            // Operand descriptors differ from stage to stage and from one 16-deep step to the next only
            // in their address field (bytes / 16): they are carried along by additions.
            const uint64_t desc0 = umma_desc(smem_u32(smem));
            const uint64_t stage_step = (uint64_t)(stage_bytes >> 4), b_step = (uint64_t)(b_off >> 4);
            const uint64_t a_atom = (uint64_t)(A_TILE_BYTES >> 4), b_atom = (uint64_t)(b_atom_bytes >> 4);
            bool ok = true;
            ItemIter iter = make_iter(g);
            Item item;
            for (; ok && iter.next(item); lt++) {
                const int n_kb = item.n_kb;
                const int buf = lt & 1;
                // the epilogue must have read this accumulator (two work items ago)
                if (!__all_sync(0xffffffffu, mbar_wait(&ctl->tmem_empty[buf], ((uint32_t)(lt >> 1) & 1u) ^ 1u, ctl, 4))) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tmem_d = tmem_base + (uint32_t)(buf * g.n_tile);
                for (int i = 0; i < n_kb; i++) {
                    if (!__all_sync(0xffffffffu, mbar_wait(&ctl->full[s], phase, ctl, 2))) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    if (elect_one()) {
                        const uint64_t a_desc = desc0 + (uint64_t)s * stage_step, b_desc = a_desc + b_step;
                        umma_bf16(tmem_d, a_desc, b_desc, idesc, i > 0 ? 1u : 0u);
#pragma unroll
                        for (int k = 1; k < BLOCK_K / UMMA_K; k++)
                            umma_bf16(tmem_d, a_desc + (uint64_t)(k * UMMA_K * 2 >> 4), b_desc + (uint64_t)(k * UMMA_K * 2 >> 4), idesc, 1u);
                        if (g.atoms == 2) {
#pragma unroll
                            for (int k = 0; k < BLOCK_K / UMMA_K; k++)
                                umma_bf16(tmem_d, a_desc + a_atom + (uint64_t)(k * UMMA_K * 2 >> 4),
                                          b_desc + b_atom + (uint64_t)(k * UMMA_K * 2 >> 4), idesc, 1u);
                        }
                        umma_commit(&ctl->empty[s]);      // frees the stage when these MMAs have read it
                    }
                    __syncwarp();
                    if (++s == g.stages) { s = 0; phase ^= 1u; }
                }
                if (ok) {
                    if (elect_one()) umma_commit(&ctl->tmem_full[buf]);   // this accumulator is complete
                    __syncwarp();
                }
            }
        }
    } else {
        // ---------------- epilogue: warps 2..5 ----------------
        const int quarter = warp & 3;                 // TMEM lanes 32*quarter .. +31 belong to this warp
        const int row = quarter * 32 + lane;          // row of the A tile
        int lt = 0;
        bool first = true;
        ItemIter iter = make_iter(g);
        Item item;
        for (; iter.next(item); lt++) {
            const int tile_b = item.tile_b, tile_a = item.tile_a;
            const int a_row = tile_a * BLOCK_M + row;
            const int buf = lt & 1;
            // every epilogue thread takes the same decision, so that all of them reach the
            // named barriers below
            if (!mbar_wait(&ctl->tmem_full[buf], (uint32_t)(lt >> 1) & 1u, ctl, 3)) atomicExch(&ctl->epi_ok, 0);
            if (first) { pdl_wait(); first = false; }     // before the first access to C, workspace, counters
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (*(volatile int*)&ctl->epi_ok == 0) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * g.n_tile);
            if (g.cluster > 1) {
                // This CTA's sums go to its own shared memory (the ring is free: every MMA that read
                // it has completed) as [column / 4][row][4]; the cluster adds them up below.
                float4* dump = reinterpret_cast<float4*>(smem);
                for (int c0 = 0; c0 < g.n_tile; c0 += 16) {
                    uint32_t r[16];
                    tmem_ld16(taddr + (uint32_t)c0, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 4; j++)
                        dump[(size_t)(c0 / 4 + j) * BLOCK_M + row] =
                            make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                        __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                cl_tile_a = tile_a; cl_tile_b = tile_b;
                break;                                      // one work item per CTA in this mode
            }
            const bool shared_tile = item.n_parts > 1;      // several work items add up to this tile
            const int tile_id = tile_a * tiles_b + tile_b;
            // A piece lies in the workspace as [column / 4][row][4] floats: a thread's four columns
            // are one 16-byte access and a warp's accesses are contiguous.
            bool fast = false;
            if (shared_tile && g.streamk) {
                // All the other pieces are there already (the usual case for the piece a CTA ends
                // its run with): add them to the accumulator without writing it out first.
                if (warp == 2 && lane == 0) {
                    int seen;
                    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(g.counters + tile_id) : "memory");
                    ctl->is_last = (seen == item.n_parts - 1) ? 1 : 0;
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                fast = *(volatile int*)&ctl->is_last != 0;
            }
            if (fast) {
                __threadfence();
                for (int c0 = 0; c0 < g.n_tile; c0 += 32) {
                    const bool two = c0 + 16 < g.n_tile;
                    float acc[32];
                    for (int sp = 0; sp < item.n_parts; sp++) {
                        float t[32];
                        if (sp == item.my_part) {
                            uint32_t r[2][16];
                            tmem_ld16(taddr + (uint32_t)c0, r[0]);
                            if (two) tmem_ld16(taddr + (uint32_t)(c0 + 16), r[1]);
                            tmem_ld_wait();
#pragma unroll
                            for (int q = 0; q < 2; q++)
#pragma unroll
                                for (int j = 0; j < 16; j++) t[16 * q + j] = __uint_as_float(r[q][j]);
                        } else {
                            const float4* src = reinterpret_cast<const float4*>(g.workspace + part_base(g, iter, item, sp)) +
                                                (size_t)(c0 / 4) * BLOCK_M + row;
#pragma unroll
                            for (int i = 0; i < 8; i++) {
                                float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
                                if (i < 4 || two) x = __ldcg(src + (size_t)i * BLOCK_M);
                                t[4 * i] = x.x; t[4 * i + 1] = x.y; t[4 * i + 2] = x.z; t[4 * i + 3] = x.w;
                            }
                        }
                        if (sp == 0) {
#pragma unroll
                            for (int j = 0; j < 32; j++) acc[j] = t[j];
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; j++) acc[j] += t[j];
                        }
                    }
#pragma unroll
                    for (int q = 0; q < 2; q++)
                        if ((q == 0 || two) && tile_b * g.n_tile + c0 + 16 * q < g.rows_b)
                            emit<16>(g, a_row, tile_b * g.n_tile + c0 + 16 * q, reinterpret_cast<const float(&)[16]>(acc[16 * q]));
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&ctl->tmem_empty[buf])) : "memory");
                if (warp == 2 && lane == 0) g.counters[tile_id] = 0;
                continue;
            }
            // 32 columns per wait (n_tile is a multiple of 16: the last group may be half)
            for (int c0 = 0; c0 < g.n_tile; c0 += 32) {
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
                    const int c = c0 + 16 * h;
                    if (shared_tile) {
                        float4* part = reinterpret_cast<float4*>(g.workspace + part_base(g, iter, item, item.my_part)) +
                                       (size_t)(c / 4) * BLOCK_M + row;
#pragma unroll
                        for (int j = 0; j < 4; j++)
                            part[(size_t)j * BLOCK_M] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                    } else {
                        emit<16>(g, a_row, tile_b * g.n_tile + c, v);
                    }
                }
            }
            // the accumulator has been read: the MMA warp may reuse it
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0 && !g.withhold_release)
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&ctl->tmem_empty[buf])) : "memory");
            if (shared_tile) {
                // the CTA that arrives last adds the partial sums in k order
                __threadfence();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (warp == 2 && lane == 0) {
                    const int old = atomicAdd(&g.counters[tile_id], 1);
                    ctl->is_last = (old == item.n_parts - 1) ? 1 : 0;
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (*(volatile int*)&ctl->is_last) {
                    __threadfence();
                    // the loads of four pieces are in flight together; the sums stay in k order
                    const float4* src4[4];
#pragma unroll
                    for (int q = 0; q < 4; q++)
                        src4[q] = reinterpret_cast<const float4*>(
                                      g.workspace + part_base(g, iter, item, q < item.n_parts ? q : 0)) + row;
                    for (int c0 = 0; c0 < g.n_tile; c0 += 16) {
                        if (tile_b * g.n_tile + c0 >= g.rows_b) break;
                        float acc[16];
                        for (int sp0 = 0; sp0 < item.n_parts; sp0 += 4) {
                            float4 t[4][4];
#pragma unroll
                            for (int q = 0; q < 4; q++) {
                                if (sp0 + q >= item.n_parts) break;
                                const float4* src = (sp0 == 0 ? src4[q]
                                                              : reinterpret_cast<const float4*>(
                                                                    g.workspace + part_base(g, iter, item, sp0 + q)) + row) +
                                                    (size_t)(c0 / 4) * BLOCK_M;
#pragma unroll
                                for (int u = 0; u < 4; u++) t[q][u] = __ldcg(src + (size_t)u * BLOCK_M);
                            }
#pragma unroll
                            for (int q = 0; q < 4; q++) {
                                if (sp0 + q >= item.n_parts) break;
#pragma unroll
                                for (int u = 0; u < 4; u++) {
                                    if (sp0 + q == 0) {
                                        acc[4 * u] = t[q][u].x; acc[4 * u + 1] = t[q][u].y;
                                        acc[4 * u + 2] = t[q][u].z; acc[4 * u + 3] = t[q][u].w;
                                    } else {
                                        acc[4 * u] += t[q][u].x; acc[4 * u + 1] += t[q][u].y;
                                        acc[4 * u + 2] += t[q][u].z; acc[4 * u + 3] += t[q][u].w;
                                    }
                                }
                            }
                        }
                        emit<16>(g, a_row, tile_b * g.n_tile + c0, acc);
                    }
                    if (warp == 2 && lane == 0) g.counters[tile_id] = 0;
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");      // is_last is rewritten by the next item
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }

    __syncthreads();
    if (g.cluster > 1) {
        // The K splits of the tile are this cluster's CTAs, in rank order.  Each CTA adds up its
        // share of the rows from all the CTAs' shared memory, always in rank order, and stores:
        // no scratch in global memory, no counter, and every SM of the cluster adds.
        cluster_sync();
        if (warp >= 2 && *(volatile int*)&ctl->abort_flag == 0 && *(volatile int*)&ctl->epi_ok) {
            const int S = g.cluster, rank = (int)cluster_rank();
            // even shares of rows: a gate row and its up row stay with neighbouring lanes (emit)
            const int r0 = rank * (BLOCK_M / 2) / S * 2, nrows = (rank + 1) * (BLOCK_M / 2) / S * 2 - r0;
            const int groups = g.n_tile / 16;
            const int t = (int)threadIdx.x - 64;
            const uint32_t base = smem_u32(smem);
            uint32_t peer[8];
#pragma unroll
            for (int q = 0; q < 8; q++) peer[q] = peer_smem(base, (uint32_t)(q < S ? q : 0));
            for (int u0 = t - lane; u0 < nrows * groups; u0 += 128) {       // whole warps call emit
                const int u = u0 + lane;
                const bool mine = u < nrows * groups;
                const int row = mine ? r0 + u % nrows : 0, grp = mine ? u / nrows : 0;
                const uint32_t off = (uint32_t)(((grp * 4) * BLOCK_M + row) * 16);
                float acc[16];
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    float4 v[4][4];
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        if (4 * h + q >= S) break;
#pragma unroll
                        for (int j = 0; j < 4; j++) v[q][j] = ld_cluster_f4(peer[4 * h + q] + off + (uint32_t)(j * BLOCK_M * 16));
                    }
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        if (4 * h + q >= S) break;
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            if (4 * h + q == 0) {
                                acc[4 * j] = v[q][j].x; acc[4 * j + 1] = v[q][j].y; acc[4 * j + 2] = v[q][j].z; acc[4 * j + 3] = v[q][j].w;
                            } else {
                                acc[4 * j] += v[q][j].x; acc[4 * j + 1] += v[q][j].y; acc[4 * j + 2] += v[q][j].z; acc[4 * j + 3] += v[q][j].w;
                            }
                        }
                    }
                }
                emit<16>(g, mine ? cl_tile_a * BLOCK_M + row : 0x3fffffff, cl_tile_b * g.n_tile + grp * 16, acc);
            }
        }
        cluster_sync();                               // nobody leaves while its shared memory is read
    }
    if (*(volatile int*)&ctl->abort_flag) {
        // a wait ran out: give copies and MMAs in flight a fixed time to land before the
        // shared and tensor memory of this CTA are released
        const unsigned long long t0 = global_ns();
        while (global_ns() - t0 < 2000000ull) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
    }
}

// ---------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------
PFN_cuTensorMapEncodeTiled_v12000 g_encode = nullptr;
// One k-block of a 128 x n_tile tile, measured with all SMs busy (2,048 x 16384 x 3072: 222, 170, 149 us at
// 128, 192, 256 columns): the wide tile is bounded by the tensor cores at the clock the power limit
// leaves, the narrow one by what the L2 delivers (32 KB per k-block and SM).
inline long long kb_ns(int n_tile) { return n_tile <= 128 ? 330 : n_tile <= 192 ? 353 : 444; }
int g_force_tile = 0;       // measurements only: tile width and schedule for many tokens (0, -1: chosen here)
int g_force_streamk = -1;
int g_force_narrow = -1;      // 48..128 tokens: 1 narrow tiles, 0 swap-AB with split K, -1 by the shape
const uint8_t* g_pf_ptr = nullptr;   // set by oe_gemm_tc_prefetch for the next launch
long long g_pf_bytes = 0;
int g_force_cluster = -1;     // 0: K splits add up through the workspace even where a cluster could
int g_force_atoms = -1;       // up to 128 tokens, swap-AB: 64-deep atoms per k-block (1 or 2; -1 by the shape)
unsigned long long g_wait_ns = WAIT_LIMIT_NS;   // the limit the next launches give their waits
int g_withhold_release = 0;   // tests: see GemmArgs::withhold_release
int g_max_clusters[9] = {-1, -1, -1, -1, -1, -1, -1, -1, -1};   // clusters of that many CTAs that fit on the GPU at once
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

// [rows, K] bf16 row-major with leading dimension ld (elements); box = BLOCK_K x box_rows
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

// Clusters of cs CTAs of the kernel that the GPU holds at once (one CTA per SM); < 0: -error.
int max_clusters(int cs) {
    if (cs < 1 || cs > 8) return 0;
    if (g_max_clusters[cs] >= 0) return g_max_clusters[cs];
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return -(int)e;
    cudaLaunchConfig_t probe = {};
    probe.gridDim = dim3((unsigned)cs); probe.blockDim = dim3(THREADS); probe.dynamicSmemBytes = 227 * 1024;
    cudaLaunchAttribute pa[1];
    pa[0].id = cudaLaunchAttributeClusterDimension;
    pa[0].val.clusterDim.x = (unsigned)cs; pa[0].val.clusterDim.y = 1; pa[0].val.clusterDim.z = 1;
    probe.attrs = pa; probe.numAttrs = 1;
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, gemm_tc_kernel, &probe);
    if (e != cudaSuccess) { cudaGetLastError(); n = 0; }
    g_max_clusters[cs] = n;
    return n;
}

}  // namespace

extern "C" {

// 1 if the tensor-core kernel takes these operands (TMA needs 16-byte aligned rows).
int oe_gemm_tc_supported(const void* A, const void* W, int M, int N, int K, long long lda) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    if ((K % 8) || (lda % 8)) return 0;
    if (((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return 0;
    return 1;
}

// Workspace bytes and counters the split-K path may need for any call with up to
// `max_tokens` rows on the swapped path.
long long oe_gemm_tc_workspace_bytes() { return 64ll << 20; }
int oe_gemm_tc_counters() { return 4096; }

// C[M,N] (+)= A[M,K] . W[N,K]^T ; out_kind: 0 bf16, 1 float32, 2 float32 accumulate,
// 3: W's rows alternate gate/up and C[M,N/2] = silu(gate) * up as bf16 (ldc counts C's elements).
// workspace: float32 scratch of ws_bytes bytes, counters: n_counters zeroed ints (both may be null: no split).
int oe_gemm_tc_bf16(void* C, const bf16* A, const bf16* W, int M, int N, int K, long long lda, long long ldc,
                    int out_kind, float* workspace, long long ws_bytes, int* counters, int n_counters,
                    int sm_count, cudaStream_t st) {
    if (!oe_gemm_tc_supported(A, W, M, N, K, lda)) return OE_ERR_UNSUPPORTED;
    if (out_kind < 0 || out_kind > 3 || (out_kind == 3 && (N & 1))) return OE_ERR_UNSUPPORTED;
    int rc = get_encode();
    if (rc) return rc;
    GemmArgs g;
    g.C = C; g.ldc = ldc; g.K = K; g.out_kind = out_kind;
    g.workspace = workspace; g.counters = counters; g.splits = 1; g.streamk = 0; g.sk_tiles = 0; g.cluster = 1;
    g.atoms = 1;
    g.wait_ns = g_wait_ns; g.withhold_release = g_withhold_release;
    g.pf_ptr = g_pf_ptr; g.pf_bytes = g_pf_bytes; g_pf_ptr = nullptr; g_pf_bytes = 0;
    CUtensorMap map_a, map_b;
    dim3 grid;
    int n_kb = (K + BLOCK_K - 1) / BLOCK_K;
    // 48..128 tokens, a short K and so many weight rows that swap-AB could not split K (fewer than
    // two CTAs per 128 rows): the activations stay the 128-row operand (rows beyond M are not
    // fetched) and a narrow weight tile per CTA gives about one CTA per SM, no split.  Measured at
    // 64 tokens: 16384x3072 27.7 us against 31.4 with swap-AB; with a split the swapped form wins
    // (5120x3072 22 -> 16 us, 3072x3072 21 -> 14 us) since its splits add up inside a cluster.
    const bool can_split = sm_count / ((N + BLOCK_M - 1) / BLOCK_M) >= 2 && workspace != nullptr;
    const bool narrow = g_force_narrow >= 0 ? (g_force_narrow == 1 && M <= 128)
                                            : (M <= 128 && M >= 48 && K <= 4096 && !can_split);
    if (narrow) {
        g.swap = 0;
        int nt = ((N + sm_count - 1) / sm_count + 15) / 16 * 16;
        if (nt < 16) nt = 16;
        if (nt > 256) nt = 256;
        g.n_tile = nt;
        g.rows_a = M; g.rows_b = N;
        g.atoms = g_force_atoms > 0 ? g_force_atoms : (K >= 1024 ? 2 : 1);    // gate/up at 64 tokens: 30.5 -> 25.6 us
        n_kb = (K + BLOCK_K * g.atoms - 1) / (BLOCK_K * g.atoms);
        if ((rc = make_map(&map_a, A, M, K, lda, BLOCK_M))) return rc;
        if ((rc = make_map(&map_b, W, N, K, K, g.n_tile))) return rc;
        g.tiles_a = 1;
        g.tiles_b = (N + g.n_tile - 1) / g.n_tile;
    } else if (M <= 128) {
        // few tokens: weights fill the 128 rows of the instruction, tokens are its N
        g.swap = 1;
        g.n_tile = ((M + 15) / 16) * 16;
        g.rows_a = N; g.rows_b = M;
        // One CTA alone on the GPU streams 38 GB/s of weights with k-blocks of one 64-deep atom
        // (24 KB a stage at 64 tokens, 417 ns each) and 53 GB/s with two atoms (48 KB, 600 ns): a
        // k-block costs about 230 ns whatever it brings, plus its bytes at about 130 GB/s.  With two
        // atoms the layer products at 64 tokens take 11.8, 13.8, 16.7 us instead of 13.0, 15.7, 19.9;
        // a product with many tiles per CTA (the logits) streams at 0.9 of the HBM figure either way.
        g.atoms = g_force_atoms > 0 ? g_force_atoms
                                    : ((K >= 1024 && (N + BLOCK_M - 1) / BLOCK_M <= 2 * sm_count) ? 2 : 1);
        n_kb = (K + BLOCK_K * g.atoms - 1) / (BLOCK_K * g.atoms);
        const int tiles_a = (N + BLOCK_M - 1) / BLOCK_M;
        int splits = 1;
        if (workspace && counters && tiles_a <= n_counters) {
            splits = sm_count / tiles_a;                      // one wave of CTAs
            if (splits > n_kb * g.atoms / 4) splits = n_kb * g.atoms / 4;
            if (splits > n_kb) splits = n_kb;
            if (splits < 1) splits = 1;
            const long long need = (long long)splits * tiles_a * g.n_tile * BLOCK_M * 4;
            if (need > ws_bytes) splits = 1;
            const int kb_per = (n_kb + splits - 1) / splits;
            splits = (n_kb + kb_per - 1) / kb_per;          // no split without work
        }
        g.splits = splits;
        // The splits of a tile as one cluster: the largest number of splits, at most 8 (the
        // portable cluster size), with which all clusters run at once (a cluster lies within one
        // GPC, so fewer clusters of 6 fit than 148 / 6).
        if (splits >= 2 && g_force_cluster != 0) {
            for (int cs = splits < 8 ? splits : 8; cs >= 2; cs--) {
                const int fit = max_clusters(cs);
                if (fit < 0) return -fit;
                if (fit < tiles_a) continue;
                const int kb_per = (n_kb + cs - 1) / cs;
                g.splits = (n_kb + kb_per - 1) / kb_per;
                g.cluster = g.splits;
                break;
            }
        }
        if ((rc = make_map(&map_a, W, N, K, K, BLOCK_M))) return rc;
        if ((rc = make_map(&map_b, A, M, K, lda, g.n_tile))) return rc;
        g.tiles_a = tiles_a; g.tiles_b = 1;
    } else {
        g.swap = 0;
        if (N < 256) {
            g.n_tile = ((N + 15) / 16) * 16;
        } else {
            // The tile width with the shortest rounds of CTAs (one CTA per SM) at the measured time of
            // a k-block (kb_ns); at 2,048 and 8,192 tokens and this model's four shapes that choice is
            // the best of the three or within 1 % of it.
            const int tiles_m = (M + BLOCK_M - 1) / BLOCK_M;
            long long best = -1;
            for (int nt = 256; nt >= 128; nt -= 64) {
                const long long tiles = (long long)tiles_m * ((N + nt - 1) / nt);
                const long long cost = ((tiles + sm_count - 1) / sm_count) * kb_ns(nt);
                if (best < 0 || cost < best) { best = cost; g.n_tile = nt; }
            }
            if (g_force_tile >= 16 && g_force_tile <= 256 && g_force_tile % 16 == 0) g.n_tile = g_force_tile;
        }
        g.rows_a = M; g.rows_b = N;
        g.tiles_a = (M + BLOCK_M - 1) / BLOCK_M;
        // Stream-K (see ItemIter) where it saves a tenth or more over whole tiles of the width
        // chosen above, and the round of whole tiles after the shared part lasts longer than
        // the adding up of a shared tile's pieces (about 10 us a piece while the other SMs
        // multiply), which then costs nothing.  (2,048 tokens: 3072 -> 5120 72 -> 68 us,
        // 8192 -> 3072 117 -> 100 us; 8,192 tokens: 8192 -> 3072 386 -> 353 us; 3072 -> 3072 at
        // 2,048 tokens stays with whole tiles: its round of whole tiles is too short, 46 -> 65 us.)
        const int sk = g_force_streamk;
        const long long tiles256 = (long long)g.tiles_a * ((N + 255) / 256);
        if (sk != 0 && N >= 256 && workspace && counters && tiles256 <= n_counters &&
            2LL * sm_count * 256 * BLOCK_M * 4 <= ws_bytes) {
            const long long tiles_now = (long long)g.tiles_a * ((N + g.n_tile - 1) / g.n_tile);
            const double whole = (double)((tiles_now + sm_count - 1) / sm_count) * (double)kb_ns(g.n_tile);
            const double shared_k = (double)tiles256 / (double)sm_count * (double)kb_ns(256);
            const long long rounds = tiles256 / sm_count, rest = tiles256 % sm_count;
            if (sk == 1 ? rest > 0 : (rounds >= 1 && rest > 0 && shared_k < 0.9 * whole)) {
                // the shared part: the remainder, plus one full round if the remainder alone would
                // cut its tiles into more than four pieces and a round of whole tiles is still left
                long long shared = rest;
                if (rounds >= 2 && rest * 4 < sm_count) shared += sm_count;
                const long long run = shared * n_kb / sm_count;
                const long long pieces = run > 0 ? (n_kb + run - 1) / run + 1 : 1000;
                if (sk == 1 ? run >= 1 : (run >= 8 && (double)pieces * 10000.0 <= (double)n_kb * (double)kb_ns(256))) {
                    g.streamk = 1;
                    g.sk_tiles = (int)shared;
                    g.n_tile = 256;
                }
            }
        }
        g.tiles_b = (N + g.n_tile - 1) / g.n_tile;
        // A few hundred tokens: tiles of 128 x 256 fill less than half of the SMs.  K is split over the CTAs
        // of a cluster per tile, as for few tokens (8192 -> 3072 at 512 tokens: 48 tiles, 3 CTAs each).
        // The caller that wants no split (workspace == nullptr) gets none.
        const long long tiles_wide = (long long)g.tiles_a * ((N + 255) / 256);
        if (!g.streamk && g_force_cluster != 0 && workspace != nullptr && N >= 256 && tiles_wide * 2 <= sm_count &&
            n_kb >= 8 && g_force_tile == 0) {
            int want = (int)(sm_count / tiles_wide);
            if (want > n_kb / 4) want = n_kb / 4;
            for (int cs = want < 8 ? want : 8; cs >= 2; cs--) {
                const int fit = max_clusters(cs);
                if (fit < 0) return -fit;
                if (fit < tiles_wide) continue;
                const int kb_per = (n_kb + cs - 1) / cs;
                g.splits = (n_kb + kb_per - 1) / kb_per;
                g.cluster = g.splits;
                g.n_tile = 256;
                g.tiles_b = (N + 255) / 256;
                break;
            }
        }
        if ((rc = make_map(&map_a, A, M, K, lda, BLOCK_M))) return rc;
        if ((rc = make_map(&map_b, W, N, K, K, g.n_tile))) return rc;
    }
    const long long n_work = (long long)g.tiles_a * g.tiles_b * g.splits;
    if (n_work > 2147483647LL) return OE_ERR_UNSUPPORTED;
    g.n_kb_total = (K + BLOCK_K * g.atoms - 1) / (BLOCK_K * g.atoms);
    g.kb_per = (g.n_kb_total + g.splits - 1) / g.splits;
    grid = dim3((unsigned)((n_work < sm_count && !g.streamk) ? n_work : sm_count));
    const int b_tile_bytes = g.n_tile * BLOCK_K * 2;
    const int stage_bytes = g.atoms * (A_TILE_BYTES + ((b_tile_bytes + 1023) & ~1023));
    int stages = (200 * 1024) / stage_bytes;
    if (stages > 10) stages = 10;
    if (stages > n_kb && n_kb > 0) stages = n_kb < 2 ? 2 : n_kb;
    if (stages < 2) stages = 2;
    g.stages = stages;
    const size_t smem = (size_t)stages * stage_bytes + sizeof(SharedCtl) + 1024;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) return (int)e;
        attr_set = true;
    }
    if (g.cluster > 1)
        return oe_launch_cluster(gemm_tc_kernel, (unsigned)g.cluster, dim3(grid), dim3(THREADS), smem, st, map_a, map_b, g);
    const int launch_rc = oe_launch(gemm_tc_kernel, dim3(grid), dim3(THREADS), smem, st, map_a, map_b, g);
    return launch_rc;
}

// For measurements: forces the tile width (0: chosen by the shape) and the schedule (1: stream-K
// wherever a remainder exists, 0: whole tiles, -1: chosen by the shape) of products over many tokens,
// (cluster = 0) K splits of few tokens through the workspace instead of a cluster, and (narrow = 1 / 0)
// up to 128 tokens narrow tiles without a split or swap-AB with split K, and (atoms = 1 / 2) how many
// 64-deep swizzle atoms a k-block of those products holds.
// The next launch asks the first `bytes` bytes at `ptr` (the weights of the product that follows it) into the L2.
void oe_gemm_tc_prefetch(const void* ptr, long long bytes) { g_pf_ptr = (const uint8_t*)ptr; g_pf_bytes = bytes > 0 ? bytes : 0; }

void oe_gemm_tc_force(int n_tile, int streamk, int cluster, int narrow, int atoms) {
    g_force_tile = n_tile; g_force_streamk = streamk; g_force_cluster = cluster; g_force_narrow = narrow;
    g_force_atoms = atoms;
}

// The limit (nanoseconds; <= 0: the default of 2 s) that the waits of the following launches get, and, for
// the test of the path a run-out wait takes, whether their epilogues withhold the release of their
// accumulators (the MMA role's wait then runs out on a CTA's third tile, the kernel sets the error flag,
// waits for what is in flight, frees its tensor memory and returns; its output is then not valid).
void oe_gemm_tc_waits(long long wait_ns, int withhold_release) {
    g_wait_ns = wait_ns > 0 ? (unsigned long long)wait_ns : WAIT_LIMIT_NS;
    g_withhold_release = withhold_release ? 1 : 0;
}

// Diagnostics: how many clusters of cs CTAs of the kernel run at once.
int oe_gemm_tc_max_clusters(int cs) { return max_clusters(cs); }

// Reads and clears the device-side error flag (0 = no wait ran out).
int oe_gemm_tc_error() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_error, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) cudaMemcpyToSymbol(g_error, &zero, sizeof(int));
    return v;
}

}  // extern "C"
