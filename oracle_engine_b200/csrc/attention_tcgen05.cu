// Causal grouped-query attention of prompts over the paged cache on the 5th-generation
// tensor cores (sm_100a), compiled for one head size: -DOE_HD=64 or 128.
//
// A CTA owns 128 query rows of one (sequence, KV head); a row is a (token, query head of
// the group) pair, so the G = H/KVH heads that share a KV head share every K/V tile.  Key
// blocks are cache pages (64 keys).  Per block:
//   S = Q K^T      tcgen05.mma M=128 N=64 K=head_dim, Q and K tiles K-major in 128B-swizzled
//                  shared memory (TMA), S float32 in tensor memory (two buffers);
//   softmax        128 threads, one row each: tcgen05.ld of the row's 64 scores, causal /
//                  window mask, maximum and sum in float32 (no shuffles: a thread holds its
//                  whole row), P = exp2(s * scale - m) rounded to bf16 and stored back into
//                  the first half of the same tensor-memory columns (tcgen05.st);
//   O += P V       tcgen05.mma M=128 N=head_dim K=64, P as the A operand from tensor memory,
//                  V as the MN-major B operand straight from the page ([key][dim] rows of 128
//                  bytes), O float32 in tensor memory for the whole tile.
// The reference maximum m of a row moves only when the row's maximum has grown by more than
// 2^8 since it was set: then the row's O (tcgen05.ld, multiply, tcgen05.st) and its sum are
// rescaled before the block's P V is issued.  Between two moves P <= 2^8, which bf16 and the
// float32 sums hold without loss, and the factor cancels in the final O / l, so the result
// is the one of the plain online softmax.  The decision is taken per warp (tensor-memory
// loads and stores are warp-wide).
// The MMA thread issues S of block j+1 before it waits for P of block j, so the tensor pipe
// and the softmax overlap; two CTAs share an SM (96 KB of shared memory, 256 columns of
// tensor memory and at most 168 registers a thread each), which hides the latencies of one
// CTA's softmax chain behind the other's.
// Roles (192 threads): warp 0 = TMA producer (Q once, then K and V pages through two-stage
// rings of their own: a K stage is free once its S is done, a V stage once its P V is done),
// warp 1 = tensor-memory allocation and MMA issue, warps 2-5 = softmax and output.
// Every wait on an mbarrier is bounded in time; a wait that runs out raises an error flag,
// every role leaves its loop, copies in flight get a fixed time, tensor memory is freed.
// Reference: core/model.cpp:605-626 (scores, softmax, weighted values of a prompt).
#include <cuda.h>
#include <cudaTypedefs.h>
#include "common.cuh"
#include <mutex>

#ifndef OE_HD
#define OE_HD 128
#endif

namespace {

constexpr int HD = OE_HD;
static_assert(HD == 64 || HD == 128, "the tcgen05 attention is built for head_dim 64 or 128");
constexpr int BM = 128;                    // query rows per CTA
constexpr int BN = OE_PAGE;                // keys per block
constexpr int SUB = HD / 64;               // 64-wide (128-byte) sub-tiles along head_dim
constexpr int Q_BYTES = BM * HD * 2;       // SUB sub-tiles of [128][64]
constexpr int KV_TILE = BN * HD * 2;       // one K or V page panel, SUB sub-tiles of [64][64]
constexpr int STAGES = 2;                  // of the K ring and of the V ring
constexpr int THREADS = 192;
constexpr uint32_t TMEM_COLS = 256;        // S: 2 x 64, O: HD
constexpr uint32_t S_COL = 0, O_COL = 128;
constexpr float RESCALE_STEP = 8.f;        // log2 units
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;

__device__ int g_error = 0;

struct Ctl {
    uint64_t q_full;
    uint64_t k_full[STAGES], k_empty[STAGES], v_full[STAGES], v_empty[STAGES];
    uint64_t s_full[2], p_ready[2], pv_done, o_done;
    uint32_t tmem_base;
    int abort_flag;
};
constexpr int SMEM_NEEDED = Q_BYTES + 2 * STAGES * KV_TILE + (int)sizeof(Ctl);

struct Args {
    bf16* out;                 // [T, H*HD]
    const int* tables;         // [B, max_pages]
    int max_pages;
    const int* cu_q;
    const int* seq_start;
    const int* seq_qlen;
    int H, KVH, window;
    float scale_log2;
    int tokens_per_tile;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
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
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
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
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, Ctl* ctl, int code) {
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
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"((uint64_t)map), "r"(smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(dst)), "l"((uint64_t)map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
// Shared-memory operand descriptor, 128-byte swizzle, version 1 (sm_100).
// K-major (rows of 128 bytes along K): stride offset 1024 between 8-row groups.
// MN-major (rows of 128 bytes along N, one row per k): stride offset 1024 between 8-k groups,
// leading offset = distance between 64-wide column groups.
__device__ __forceinline__ uint64_t umma_desc(uint32_t addr, uint32_t lead_bytes, uint32_t stride_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)((lead_bytes >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((stride_bytes >> 4) & 0x3FFFu) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// kind::f16 instruction descriptor: D float32, A and B bf16, A K-major, B K-major or MN-major.
__device__ __forceinline__ uint32_t umma_idesc(int m, int n, bool b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// The same with the A operand in tensor memory (rows = lanes, two bf16 of consecutive k per column).
__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// 16 columns of this thread's TMEM lane; the values are valid after tmem_ld_wait().
__device__ __forceinline__ void tmem_ld16_nowait(uint32_t taddr, float* v) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]), "=f"(v[6]), "=f"(v[7]),
          "=f"(v[8]), "=f"(v[9]), "=f"(v[10]), "=f"(v[11]), "=f"(v[12]), "=f"(v[13]), "=f"(v[14]), "=f"(v[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const float* v) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
          "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
          "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
          "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15]))
        : "memory");
}
__device__ __forceinline__ void tmem_st16_u32(uint32_t taddr, const uint32_t* v) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
          "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// True in exactly one lane of a converged warp.  The warp stays converged around the
// instructions that lane issues, so their operands can stay in uniform registers.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__global__ void __launch_bounds__(THREADS, 2)
attn_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv, const Args a) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    {   // the swizzled tiles need a 1024-byte boundary; the launch leaves less than 1024 bytes of slack
        uint32_t dyn;
        asm volatile("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn));
        if ((uint32_t)(smem - smem_raw) + (uint32_t)SMEM_NEEDED > dyn) {
            if (threadIdx.x == 0) atomicCAS(&g_error, 0, 9);
            return;
        }
    }
    uint8_t* q_s = smem;
    uint8_t* k_s = q_s + Q_BYTES;
    uint8_t* v_s = k_s + STAGES * KV_TILE;
    Ctl* ctl = (Ctl*)(v_s + STAGES * KV_TILE);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // grid (KV heads, sequences, tiles): CTAs start in that order, so the heaviest tiles (the late rows
    // of a causal prompt) of every head and sequence start first and the light ones fill the gaps
    const int b = blockIdx.y, kvh = blockIdx.x;
    if (threadIdx.x == 0) {
        mbar_init(&ctl->q_full, 1);
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&ctl->k_full[s], 1); mbar_init(&ctl->k_empty[s], 1);
            mbar_init(&ctl->v_full[s], 1); mbar_init(&ctl->v_empty[s], 1);
        }
        mbar_init(&ctl->s_full[0], 1); mbar_init(&ctl->s_full[1], 1);
        mbar_init(&ctl->p_ready[0], 4); mbar_init(&ctl->p_ready[1], 4);   // one arrival per softmax warp; one barrier per
                                                           // S buffer: a warp may be a block ahead of the others
        mbar_init(&ctl->pv_done, 1);
        mbar_init(&ctl->o_done, 1);
        ctl->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl->tmem_base)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *(volatile uint32_t*)&ctl->tmem_base;

    pdl_launch_dependents();
    pdl_wait();                                            // q, the cache and the step's integers come from earlier kernels

    // heavy tiles (late rows of a causal prompt) first
    const int qlen = a.seq_qlen[b];
    const int tpt = a.tokens_per_tile;
    const int q_tile = (int)gridDim.z - 1 - (int)blockIdx.z;
    const bool active = qlen > 0 && q_tile * tpt < qlen;
    int n_blocks = 0, j_lo = 0, t0 = 0, nt = 0, start = 0;
    long long packed0 = 0;
    const int G = a.H / a.KVH;
    if (active) {
        start = a.seq_start[b];
        t0 = q_tile * tpt;
        nt = min(tpt, qlen - t0);
        const int pos_lo = start + t0, pos_hi = start + t0 + nt - 1;
        const int key_lo = a.window > 0 ? max(0, pos_lo - a.window + 1) : 0;
        j_lo = key_lo / BN;
        n_blocks = pos_hi / BN - j_lo + 1;
        packed0 = a.cu_q[b] + t0;
    }
    const int* trow = a.tables + (size_t)b * a.max_pages;

    if (warp == 0) {
        // ---------------- TMA producer: Q, K_0, then K_{i+1} and V_i in turn ----------------
        if (lane == 0 && active) {
            mbar_expect_tx(&ctl->q_full, (uint32_t)(SUB * tpt * G * 128));
            for (int sb = 0; sb < SUB; sb++)
                tma_load_3d(q_s + sb * (BM * 128), &map_q, &ctl->q_full, sb * 64, kvh * G, (int)packed0);
            auto load = [&](int i, int which, uint64_t* full, uint64_t* empty, uint8_t* ring, int code) -> bool {
                const int s = i % STAGES;
                if (!mbar_wait(&empty[s], ((uint32_t)(i / STAGES) & 1u) ^ 1u, ctl, code)) return false;
                const int page = trow[j_lo + i];
                const int row = ((page * 2 + which) * a.KVH + kvh) * BN;
                uint8_t* dst = ring + (size_t)s * KV_TILE;
                mbar_expect_tx(&full[s], (uint32_t)KV_TILE);
                for (int sb = 0; sb < SUB; sb++) tma_load_2d(dst + sb * (BN * 128), &map_kv, &full[s], sb * 64, row);
                return true;
            };
            bool ok = n_blocks > 0 && load(0, 0, ctl->k_full, ctl->k_empty, k_s, 1);
            for (int i = 0; i < n_blocks && ok; i++) {
                if (i + 1 < n_blocks) ok = load(i + 1, 0, ctl->k_full, ctl->k_empty, k_s, 1);
                if (ok) ok = load(i, 1, ctl->v_full, ctl->v_empty, v_s, 10);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issue ----------------
        // The whole warp runs the loop and waits; one elected lane issues.  (With the role inside
        // `if (lane == 0)` every operand of every instruction went through that one lane's registers.)
        if (active) {
            const uint32_t idesc_s = umma_idesc(BM, BN, false);
            const uint32_t idesc_o = umma_idesc(BM, HD, true);
            // every lane waits, and all take the same decision
            auto wait_all = [&](uint64_t* bar, uint32_t parity, int code) -> bool {
                return __all_sync(0xffffffffu, mbar_wait(bar, parity, ctl, code));
            };
            bool ok = wait_all(&ctl->q_full, 0, 2);
            // Operand descriptors differ from stage to stage and from one 16-deep step to the next only in
            // their address field (bytes / 16): built once, carried along by additions.
            const uint64_t q_desc = umma_desc(smem_u32(q_s), 16, 1024), k_desc = umma_desc(smem_u32(k_s), 16, 1024);
            const uint64_t v_desc = umma_desc(smem_u32(v_s), BN * 128, 1024);
            auto issue_s = [&](int i) {                       // S_i = Q K_i^T into S buffer i & 1
                const int s = i % STAGES;
                const uint64_t kd = k_desc + (uint64_t)(s * (KV_TILE >> 4));
                const uint32_t s_tmem = tmem_base + S_COL + (uint32_t)((i & 1) * BN);
                if (elect_one()) {
#pragma unroll
                    for (int k = 0; k < HD / 16; k++) {
                        const uint32_t sb = k / 4, kk = k % 4;
                        umma(s_tmem, q_desc + (uint64_t)((sb * (BM * 128) + kk * 32) >> 4),
                             kd + (uint64_t)((sb * (BN * 128) + kk * 32) >> 4), idesc_s, k > 0 ? 1u : 0u);
                    }
                    umma_commit(&ctl->s_full[i & 1]);
                    umma_commit(&ctl->k_empty[s]);           // K_i is no longer needed
                }
                __syncwarp();
            };
            if (ok && n_blocks > 0) {
                ok = wait_all(&ctl->k_full[0], 0, 3);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (ok) issue_s(0);
            }
            for (int i = 0; i < n_blocks && ok; i++) {
                if (i + 1 < n_blocks) {
                    // S buffer (i + 1) & 1 held block i - 1, read before P_{i-1} was signalled
                    const int s1 = (i + 1) % STAGES;
                    ok = wait_all(&ctl->k_full[s1], (uint32_t)((i + 1) / STAGES) & 1u, 3);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    issue_s(i + 1);
                }
                // P_i is in tensor memory, S_i has been read, O has been rescaled if it had to be
                ok = wait_all(&ctl->p_ready[i & 1], (uint32_t)(i >> 1) & 1u, 4);
                if (!ok) break;
                const int s = i % STAGES;
                ok = wait_all(&ctl->v_full[s], (uint32_t)(i / STAGES) & 1u, 5);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t vd = v_desc + (uint64_t)(s * (KV_TILE >> 4));
                // P_i sits in the first 32 columns of S buffer i & 1: 16 keys = 8 columns per instruction
                const uint32_t p_tmem = tmem_base + S_COL + (uint32_t)((i & 1) * BN);
                if (elect_one()) {
#pragma unroll
                    for (int k = 0; k < BN / 16; k++) {
                        umma_ts(tmem_base + O_COL, p_tmem + (uint32_t)(k * 8), vd + (uint64_t)((k * (16 * 128)) >> 4), idesc_o,
                                (i > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(&ctl->pv_done);
                    umma_commit(&ctl->v_empty[s]);           // V_i is no longer needed
                    if (i == n_blocks - 1) umma_commit(&ctl->o_done);   // O is complete
                }
                __syncwarp();
            }
        }
    } else {
        // ---------------- softmax and output: warps 2..5, one row per thread ----------------
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;                 // row of the tile = TMEM lane
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
        const int tok = r / G, head = kvh * G + r % G;
        const bool valid = active && tok < nt;
        const int pos = start + t0 + tok;
        float m_run = -INFINITY, l_run = 0.f;              // m_run in units of the scaled scores (log2)
        bool ok = true;
        for (int i = 0; i < n_blocks && active; i++) {
            ok = mbar_wait(&ctl->s_full[i & 1], (uint32_t)(i >> 1) & 1u, ctl, 6);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            float s[BN];
#pragma unroll
            for (int c0 = 0; c0 < BN; c0 += 16) tmem_ld16_nowait(lane_addr + S_COL + (uint32_t)((i & 1) * BN + c0), &s[c0]);
            tmem_ld_wait();
            const int key0 = (j_lo + i) * BN;
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            // A block that lies wholly before a row's position and inside its window needs no mask.  The
            // decision is the warp's: rows past the tile's tokens (a tile of 128 rows holds 126 rows of
            // 42 tokens x 3 heads, and a prompt's last tile fewer) take the unmasked path with whatever
            // their scores are, since every row's maximum, sum and output are that row's own and those
            // rows are never stored; left to each row, one such row made its warp run both paths.
            const bool needs_mask = valid && !(key0 + BN - 1 <= pos && (a.window <= 0 || key0 > pos - a.window));
            if (!__any_sync(0xffffffffu, needs_mask)) {
#pragma unroll
                for (int c = 0; c < BN; c++) mx4[c & 3] = fmaxf(mx4[c & 3], s[c]);
            } else {
                // keys key0 + c with lo <= c <= hi stay (one unsigned comparison per score)
                const int hi = valid ? min(pos - key0, BN - 1) : -1;
                const int lo = a.window > 0 ? max(pos - a.window + 1 - key0, 0) : 0;
                const unsigned span = hi >= lo ? (unsigned)(hi - lo) : 0u;
                const bool any = hi >= lo;
#pragma unroll
                for (int c = 0; c < BN; c++) {
                    const bool keep = any && (unsigned)(c - lo) <= span;
                    s[c] = keep ? s[c] : -INFINITY;
                    mx4[c & 3] = fmaxf(mx4[c & 3], s[c]);
                }
            }
            const float m_new = fmaxf(m_run, fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * a.scale_log2);
            if (i == 0) {
                m_run = m_new;
            } else if (__any_sync(0xffffffffu, valid && m_new > m_run + RESCALE_STEP)) {
                // (only the tile's own rows vote: the scores of the rows past them are whatever shared memory held)
                // P_{i-1} V_{i-1} must have been added to O before O is rescaled.  S_i is complete, so
                // P_{i-2} V_{i-2} (issued before it) is too: the parity cannot be that of an earlier block
                ok = mbar_wait(&ctl->pv_done, (uint32_t)(i - 1) & 1u, ctl, 7);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const float alpha = fast_exp2(m_run - (m_new == -INFINITY ? 0.f : m_new));
#pragma unroll
                for (int c0 = 0; c0 < HD; c0 += 16) {
                    float ob[16];
                    tmem_ld16_nowait(lane_addr + O_COL + (uint32_t)c0, ob);
                    tmem_ld_wait();
#pragma unroll
                    for (int d = 0; d < 16; d++) ob[d] *= alpha;
                    tmem_st16(lane_addr + O_COL + (uint32_t)c0, ob);
                }
                tmem_st_wait();
                l_run *= alpha;
                m_run = m_new;
            }
            const float neg_m = (m_run == -INFINITY) ? 0.f : -m_run;
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
            // P row: 64 bf16, two per column, into the first 32 columns of this S buffer (the scores
            // are in registers by now); the tensor core reads it from there as the A operand of P V
            uint32_t w[BN / 2];
#pragma unroll
            for (int c = 0; c < BN / 2; c++) {
                const float p0 = fast_exp2(fmaf(s[2 * c], a.scale_log2, neg_m));
                const float p1 = fast_exp2(fmaf(s[2 * c + 1], a.scale_log2, neg_m));
                sum4[c & 3] += p0 + p1;
                __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
                w[c] = *(uint32_t*)&h;
            }
            tmem_st16_u32(lane_addr + S_COL + (uint32_t)((i & 1) * BN), w);
            tmem_st16_u32(lane_addr + S_COL + (uint32_t)((i & 1) * BN + 16), w + 16);
            tmem_st_wait();
            l_run += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctl->p_ready[i & 1]);
        }
        if (ok && active && n_blocks > 0) {
            // a barrier of its own: the threads do not follow every phase of pv_done, so its parity
            // could be that of an earlier block
            ok = mbar_wait(&ctl->o_done, 0, ctl, 8);
            if (ok) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
                bf16* dst = a.out + (packed0 + tok) * (long long)(a.H * HD) + (size_t)head * HD;
#pragma unroll
                for (int c0 = 0; c0 < HD; c0 += 32) {
                    float ob[32];
                    tmem_ld16_nowait(lane_addr + O_COL + (uint32_t)c0, ob);
                    tmem_ld16_nowait(lane_addr + O_COL + (uint32_t)(c0 + 16), ob + 16);
                    tmem_ld_wait();
                    if (valid) {
#pragma unroll
                        for (int c = 0; c < 32; c += 8) {
                            uint32_t w[4];
#pragma unroll
                            for (int e = 0; e < 4; e++) {
                                __nv_bfloat162 h = __floats2bfloat162_rn(ob[c + 2 * e] * inv, ob[c + 2 * e + 1] * inv);
                                w[e] = *(uint32_t*)&h;
                            }
                            *(uint4*)(dst + c0 + c) = make_uint4(w[0], w[1], w[2], w[3]);
                        }
                    }
                }
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }

    __syncthreads();
    if (*(volatile int*)&ctl->abort_flag) {
        const unsigned long long t0w = global_ns();
        while (global_ns() - t0w < 2000000ull) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
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

}  // namespace

extern "C" {

int oe_attn_tc_head_dim() { return HD; }

// Prompt attention.  q: rows of q_stride bf16 with head h at h*HD (the fused qkv buffer after
// rotation); cache: one entry [pages][2][KVH][64][HD]; out [T, H*HD].  Needs 16-byte aligned
// rows (q_stride a multiple of 8) and G = H/KVH <= 128.
int oe_attn_tc_bf16(bf16* out, const bf16* q, long long q_stride, const bf16* cache, long long n_pages, const int* tables,
                    int max_pages, const int* cu_q, const int* seq_start, const int* seq_qlen, int n_seqs, int n_tokens,
                    int max_qlen, int H, int KVH, int window, float scale, cudaStream_t st) {
    if (n_seqs <= 0 || n_tokens <= 0) return 0;
    if (H % KVH || (q_stride % 8) || ((uintptr_t)q & 15) || ((uintptr_t)cache & 15) || ((uintptr_t)out & 15)) return OE_ERR_UNSUPPORTED;
    const int G = H / KVH;
    if (G > BM || n_seqs > 65535) return OE_ERR_UNSUPPORTED;
    int rc = get_encode();
    if (rc) return rc;
    Args a;
    a.out = out; a.tables = tables; a.max_pages = max_pages; a.cu_q = cu_q; a.seq_start = seq_start; a.seq_qlen = seq_qlen;
    a.H = H; a.KVH = KVH; a.window = window; a.scale_log2 = scale * 1.4426950408889634f;
    a.tokens_per_tile = BM / G;
    CUtensorMap map_q, map_kv;
    {   // q as [token][head][dim]; a box holds 64 dims of the G heads of tokens_per_tile tokens
        cuuint64_t dims[3] = {(cuuint64_t)HD, (cuuint64_t)H, (cuuint64_t)n_tokens};
        cuuint64_t strides[2] = {(cuuint64_t)HD * 2, (cuuint64_t)q_stride * 2};
        cuuint32_t box[3] = {64, (cuuint32_t)G, (cuuint32_t)a.tokens_per_tile};
        cuuint32_t es[3] = {1, 1, 1};
        CUresult r = g_encode(&map_q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<bf16*>(q), dims, strides, box, es,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return 1000 + (int)r;
    }
    {   // the cache entry as rows of HD: [pages * 2 * KVH * 64][HD]; a box is 64 rows x 64 dims
        cuuint64_t dims[2] = {(cuuint64_t)HD, (cuuint64_t)n_pages * 2 * KVH * BN};
        cuuint64_t strides[1] = {(cuuint64_t)HD * 2};
        cuuint32_t box[2] = {64, (cuuint32_t)BN};
        cuuint32_t es[2] = {1, 1};
        CUresult r = g_encode(&map_kv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<bf16*>(cache), dims, strides, box, es,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return 2000 + (int)r;
    }
    const int tiles = (max_qlen + a.tokens_per_tile - 1) / a.tokens_per_tile;
    if (tiles > 65535) return OE_ERR_UNSUPPORTED;
    // two CTAs an SM; the kernel checks that its tiles fit behind the 1024-byte boundary it needs
    const size_t smem = (size_t)SMEM_NEEDED + 1024;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        e = cudaFuncSetAttribute(attn_tc_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
        if (e != cudaSuccess) return (int)e;
        attr_set = true;
    }
    return oe_launch(attn_tc_kernel, dim3(KVH, n_seqs, tiles), dim3(THREADS), smem, st, map_q, map_kv, a);
}

int oe_attn_tc_error() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_error, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) cudaMemcpyToSymbol(g_error, &zero, sizeof(int));
    return v;
}

}  // extern "C"
