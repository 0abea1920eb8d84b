// Persistent matrix multiply for sm_100a: C[b] = act(A[b] . B[b]^T-layout + add1 + add2) with a dense
// row-major C.  Two operand types, one kernel template: f32 storage with TF32 operands (kind::tf32, 32-element
// K blocks) and f16 storage (kind::f16, 64-element K blocks, f32 accumulation, the result rounded to f16 once in
// the epilogue; an extension, the reference's IR has no half type).  A K block is 128 bytes of either, so
// the pipeline, the shared-memory layout and the operand descriptors are the same.
//
// Compared with the one-tile-per-CTA kernel in contract_tc.cu, a CTA here stays on its SM and walks over
// output tiles, and tensor memory holds TWO accumulators: while the four epilogue warps drain tile i
// (tcgen05.ld -> addends / activation -> swizzled staging tile in shared memory -> bulk tensor store),
// the producer is already loading and the MMA thread already multiplying tile i + 1.  For the short-K
// shapes of transformer layers (K = 768: 24 K-blocks per tile) fill and drain were most of a tile's time.
//
//   warp 0 lane 0   TMA producer: per K block the 128 x 32 A tile and the BN x 32 B tile (K-major, 128-byte
//                   swizzle, rounded to TF32 by the copy engine), ring of stages with full / empty mbarriers
//   warp 1 lane 0   MMA issuer: four tcgen05.mma.kind::tf32 (K = 8) per stage into accumulator `tile & 1`;
//                   waits for that accumulator to be drained, signals it full with tcgen05.commit
//   warps 2..5      epilogue: thread <-> accumulator lane <-> output row; 32 columns at a time
//
// Large matmuls with a long reduction run on CTA PAIRS (template parameter PAIR, clusters of two): `cta_group::2`
// instructions compute a 256 x BN tile on two SMs, each CTA loading its own 128 rows of A and half of B (see the
// helpers in front of the kernel).  Same instructions in the same K order: results are bit-identical to one CTA per tile.
//
// Tiles are walked column-block-major (all row blocks of one column block before the next), so the CTAs
// that run at the same time share a B tile in L2.  Row and column tails are the copy engine's zero fill
// (loads) and clipping (stores).  Every mbarrier wait is bounded as in the other tensor-core kernels.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <mutex>

#include "../tc.h"
#include "tc_host.h"
#include "tc_ptx.cuh"
#include "epilogue.cuh"
#include "launch.cuh"

namespace kn {

namespace {

using namespace tcp;

constexpr int kGpThreads = 192;
constexpr int kGpBlockM = 128;
constexpr int kGpBlockK = 32;
constexpr int kGpATileBytes = kGpBlockM * 128;
constexpr int kGpClockTiles = 16;
constexpr int kGpStageTileBytes = 128 * 128;   // epilogue staging: 128 rows x 32 columns of f32

struct GemmPersistentParams {
    int32_t bn, stages, k_iters;
    int32_t a_batch, b_batch;        // 1, or 0 when every batch entry uses the same A / B (batch stride 0)
    int32_t splits, k_iters_slice;   // split K: slice sp of a tile covers K blocks [sp * k_iters_slice, ...) and is stored
                                     // as matrix `batch * splits + sp` of the output map (the partial-sum buffer)
    int32_t m_tiles, n_tiles, batch, total_tiles;
    int64_t m, n;
    const float* add1;
    const float* add2;
    int64_t s1[3], s2[3];            // (batch, row, col) strides of the addends
    int32_t add1_mode, add2_mode;    // 0 absent, 1 one value per column, 2 a value per element (row-contiguous), 4 one value per row
    int32_t act;
    // implicit convolution operand (GemmParams::conv_operand): which operand, 32-channel blocks per filter tap,
    // filter width, padding, output width
    int32_t conv_operand, conv_cblocks, conv_s, conv_pad_y, conv_pad_x, conv_ow;
    // 4-D operands (GemmOperand4D): kd as a shift (0: the K offset is not split), rd, bi; enabled when rd > 0
    int32_t a4_kd_shift, a4_rd, a4_bi, b4_kd_shift, b4_rd, b4_bi;
    int32_t out_half;                // f16 storage and no split: the output tile is f16 (else f32: plain C or partial sums)
    uint32_t* status;
    volatile uint32_t* dbg;          // null, or 8 progress words in pinned host memory (KN_FLAG_TRACE_GEMM)
    long long* clocks;               // KN_GEMM_CLOCKS only: 8 clock64 stamps per tile of CTA 0, in pinned host memory
};

// Post-mortem aid: with KN_FLAG_TRACE_GEMM the first CTA records how far each role got (words: 0 kernel entered,
// 1 K blocks requested, 2 K blocks landed, 3 K blocks multiplied, 4 accumulator seen by the epilogue, 5 chunks
// stored, 6 epilogue done) in pinned host memory, which the host can still read after a fault has taken the
// context.  Off (null pointer) in normal operation.
__device__ __forceinline__ void dbg_mark(const GemmPersistentParams& p, uint32_t slot, uint32_t value) {
    if (p.dbg != nullptr && blockIdx.x == 0) {
        p.dbg[slot] = value;
        __threadfence_system();
    }
}

__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4}], [%1];"
                 ::"l"(map), "r"(src), "r"(c0), "r"(c1), "r"(c2)
                 : "memory");
}

__device__ __forceinline__ void mbar_arrive_local(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// ---- CTA pairs (PAIR): two CTAs of a cluster compute one 256 x BN tile with `cta_group::2` instructions.  Each
// CTA loads its own 128 rows of A and HALF of the B tile; the tensor cores of both SMs read both halves, so every SM's
// shared-memory pipe carries a third fewer bytes per multiply-add than with one CTA per tile (that pipe, not the
// tensor pipe, bounds the one-CTA kernel at about 0.83 of the tensor rate).  CTA 0 of the pair (the leader) issues the
// MMAs; the loads of both CTAs complete on the leader's barriers; `tcgen05.commit` reaches the barriers of both.
template <bool HALF, bool PAIR>   // operand storage: f16 (kind::f16) or f32 (kind::tf32); one CTA per tile or a CTA pair
__global__ void __launch_bounds__(kGpThreads, 1)
gemm_persistent_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                       const __grid_constant__ CUtensorMap map_c, const __grid_constant__ GemmPersistentParams p) {
    extern __shared__ uint8_t smem_raw[];
    constexpr int kBlockKElems = HALF ? 64 : 32;   // elements per 128-byte K block
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
    const int stages = p.stages;
    const uint32_t rank = PAIR ? cluster_rank() : 0u;           // 0: the pair's leader
    const int worker = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x, n_workers = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
    const int b_rows = PAIR ? p.bn / 2 : p.bn;                   // rows of the B tile this CTA loads
    const uint32_t b_tile_bytes = (uint32_t)b_rows * 128u;
    const uint32_t stage_bytes = kGpATileBytes + b_tile_bytes;
    const uint32_t staging_base = base + (uint32_t)stages * stage_bytes;          // two staging tiles
    const uint32_t bar_base = staging_base + 2u * kGpStageTileBytes;
    const uint32_t full_bar = bar_base, empty_bar = bar_base + 8u * stages;
    const uint32_t acc_full = bar_base + 16u * stages, acc_empty = acc_full + 16u;
    const uint32_t slot_addr = acc_empty + 16u;
    volatile uint32_t* tmem_slot = (volatile uint32_t*)(gen_base + (slot_addr - base));
    volatile int* abandon = (volatile int*)(gen_base + (slot_addr + 4u - base));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; s++) {
            mbar_init(full_bar + 8u * s, 1);
            mbar_init(empty_bar + 8u * s, 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(acc_full + 8u * b, 1);
            mbar_init(acc_empty + 8u * b, PAIR ? 256 : 128);   // (pair: the epilogue threads of both CTAs arrive on the leader's)
        }
        *abandon = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (PAIR) cluster_sync_all();   // the peer's barriers are initialised before anything is sent to them
    const uint32_t tmem_cols = 2u * (uint32_t)p.bn <= 32u ? 32u : (2u * (uint32_t)p.bn <= 64u ? 64u : (2u * (uint32_t)p.bn <= 128u ? 128u : (2u * (uint32_t)p.bn <= 256u ? 256u : 512u)));
    if (warp == 0) {
        if (PAIR) {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_addr), "r"(tmem_cols) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_addr), "r"(tmem_cols) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    asm volatile("griddepcontrol.wait;" ::: "memory");   // nothing above touches global memory

    // tile t -> (row block, column block, batch): row blocks fastest
    auto tile_coords = [&](int t, int& mt, int& nt, int& bt, int& sp) {
        mt = t % p.m_tiles;
        const int r = t / p.m_tiles;
        nt = r % p.n_tiles;
        const int r2 = r / p.n_tiles;
        sp = r2 % p.splits;
        bt = r2 / p.splits;
    };
    auto slice_blocks = [&](int sp) { return min(p.k_iters_slice, p.k_iters - sp * p.k_iters_slice); };

    if (threadIdx.x == 0) dbg_mark(p, 0, 1);
    if (warp == 0 && lane == 0) {
        // ---------------- producer
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
        int s = 0, round = 0;
        bool ok = true;
        for (int t = worker; t < p.total_tiles && ok; t += n_workers) {
            int mt, nt, bt, sp;
            tile_coords(t, mt, nt, bt, sp);
            const int k_begin = sp * p.k_iters_slice, k_end = k_begin + slice_blocks(sp);
            const int a_row0 = (PAIR ? 2 * mt + (int)rank : mt) * kGpBlockM;   // this CTA's rows of A
            const int b_row0 = nt * p.bn + (PAIR ? (int)rank * b_rows : 0);      // and of B (a pair: its half)
            // Everything about an operand read in place that does not change along K is worked out here, and what does
            // (the filter tap of a K block) is stepped, not divided: this loop runs once per K block in ONE thread,
            // and three integer divisions by run-time values in it cost more than the four MMAs of the block
            // (measured: a 3x3 convolution over 320 channels ran at 800 cycles per K block instead of 320).
            int conv_cb = 0, conv_tx = 0, conv_ty = 0, conv_row0 = 0;
            if (p.conv_operand != 0) {
                const int tap = k_begin / p.conv_cblocks;
                conv_cb = k_begin - tap * p.conv_cblocks;
                conv_ty = tap / p.conv_s;
                conv_tx = tap - conv_ty * p.conv_s;
                conv_row0 = (p.conv_operand == 1 ? a_row0 : b_row0) / p.conv_ow;
            }
            int a4_c1 = 0, a4_c2 = 0, a4_c3 = 0, b4_c1 = 0, b4_c2 = 0, b4_c3 = 0;
            if (p.a4_rd > 0) a4_c1 = a_row0 % p.a4_rd, a4_c2 = bt % p.a4_bi, a4_c3 = a_row0 / p.a4_rd + bt / p.a4_bi;
            if (p.b4_rd > 0) b4_c1 = b_row0 % p.b4_rd, b4_c2 = bt % p.b4_bi, b4_c3 = b_row0 / p.b4_rd + bt / p.b4_bi;
            for (int k = k_begin; k < k_end; k++) {
                if (round > 0 && !mbar_wait(empty_bar + 8u * s, (uint32_t)((round & 1) ^ 1), abandon, p.status, 21)) { ok = false; break; }
                const uint32_t bar = full_bar + 8u * s;
                const uint32_t dst = base + (uint32_t)s * stage_bytes;
                // pair: both CTAs' tiles complete on the LEADER's barrier, which expects the bytes of both
                if (!PAIR || rank == 0) mbar_expect_tx(bar, PAIR ? 2u * stage_bytes : stage_bytes);
                const uint32_t to_bar = PAIR ? map_to_cta(bar, 0) : bar;
                auto load3 = [&](uint32_t d, const CUtensorMap* map, int c0, int c1, int c2) {
                    if (PAIR) tma_load_3d_pair(d, map, to_bar, c0, c1, c2);
                    else tma_load_3d(d, map, to_bar, c0, c1, c2);
                };
                auto load4 = [&](uint32_t d, const CUtensorMap* map, int c0, int c1, int c2, int c3) {
                    if (PAIR) tma_load_4d_pair(d, map, to_bar, c0, c1, c2, c3);
                    else tma_load_4d(d, map, to_bar, c0, c1, c2, c3);
                };
                if (p.conv_operand != 0) {
                    // K block k = (filter tap, 32-channel block); the tile's rows are whole output rows of image `bt`,
                    // so the operand tile is one box of the image tensor (channel, x, y, image) moved by the tap:
                    // positions outside the image are the copy engine's zero fill
                    if (p.conv_operand == 1) {
                        load4(dst, &map_a, conv_cb * 32, conv_tx - p.conv_pad_x, conv_row0 + conv_ty - p.conv_pad_y, bt);
                        load3(dst + kGpATileBytes, &map_b, k * kBlockKElems, b_row0, bt * p.b_batch);
                    } else {
                        load3(dst, &map_a, k * kBlockKElems, a_row0, bt * p.a_batch);
                        load4(dst + kGpATileBytes, &map_b, conv_cb * 32, conv_tx - p.conv_pad_x, conv_row0 + conv_ty - p.conv_pad_y, bt);
                    }
                    if (++conv_cb == p.conv_cblocks) {
                        conv_cb = 0;
                        if (++conv_tx == p.conv_s) { conv_tx = 0; conv_ty++; }
                    }
                } else {
                    // (a head split or merge read in place: the tile's coordinates in the 4-D source, see GemmOperand4D;
                    // the row part does not change along K)
                    const int k0 = k * kBlockKElems;
                    if (p.a4_rd > 0) {
                        const int kh = p.a4_kd_shift ? (k0 >> p.a4_kd_shift) : 0;
                        load4(dst, &map_a, k0 - (kh << p.a4_kd_shift), a4_c1, kh + a4_c2, a4_c3);
                    } else {
                        load3(dst, &map_a, k0, a_row0, bt * p.a_batch);
                    }
                    if (p.b4_rd > 0) {
                        const int kh = p.b4_kd_shift ? (k0 >> p.b4_kd_shift) : 0;
                        load4(dst + kGpATileBytes, &map_b, k0 - (kh << p.b4_kd_shift), b4_c1, kh + b4_c2, b4_c3);
                    } else {
                        load3(dst + kGpATileBytes, &map_b, k0, b_row0, bt * p.b_batch);
                    }
                }
                dbg_mark(p, 1, (uint32_t)(k + 1));
                if (++s == stages) { s = 0; round++; }
            }
        }
    } else if (warp == 1 && lane == 0 && PAIR && rank != 0) {
        // the peer issues no MMAs (the leader's instructions drive both tensor cores)
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    } else if (warp == 1 && lane == 0) {
        // ---------------- MMA issuer
        // instruction descriptor: f32 accumulate; A and B formats 2 = TF32 (kind::tf32) or 0 = F16 (kind::f16); both
        // K-major; N, M
        const uint32_t fmt = HALF ? 0u : 2u;
        const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(p.bn >> 3) << 17) |
                               ((uint32_t)((PAIR ? 2 * kGpBlockM : kGpBlockM) >> 4) << 24);
        int s = 0, round = 0, local = 0;
        bool ok = true;
        for (int t = worker; t < p.total_tiles && ok; t += n_workers, local++) {
            const int buf = local & 1;
            const bool clk = p.clocks != nullptr && blockIdx.x == 0 && local < kGpClockTiles;
            if (clk) p.clocks[local * 8 + 0] = clock64();
            // the epilogue has drained this accumulator (its previous use was tile local - 2)
            if (local >= 2 && !mbar_wait(acc_empty + 8u * buf, (uint32_t)(((local >> 1) - 1) & 1), abandon, p.status, 22)) break;
            tc_fence_after();
            if (clk) p.clocks[local * 8 + 1] = clock64();
            const uint32_t acc = tmem_base + (uint32_t)(buf * p.bn);
            int mt, nt, bt, sp;
            tile_coords(t, mt, nt, bt, sp);
            const int k_count = slice_blocks(sp);
            // last tile of this CTA: the next kernel of the stream may be scheduled (once every CTA says so)
            if (t + n_workers >= p.total_tiles) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
            for (int k = 0; k < k_count; k++) {
                if (!mbar_wait(full_bar + 8u * s, (uint32_t)(round & 1), abandon, p.status, 23)) { ok = false; break; }
                if (clk && k == 0) p.clocks[local * 8 + 2] = clock64();
                dbg_mark(p, 2, (uint32_t)(k + 1));
                tc_fence_after();
                const uint32_t a_addr = base + (uint32_t)s * stage_bytes;
                const uint64_t da = smem_desc_sw128(a_addr);
                const uint64_t db = smem_desc_sw128(a_addr + kGpATileBytes);
                // four instructions of 32 bytes of K each: the start address advances by 2 (16-byte units)
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    if (PAIR) mma_pair<HALF>(acc, da + 2u * j, db + 2u * j, idesc, (k | j) != 0 ? 1u : 0u);
                    else if (HALF) mma_f16(acc, da + 2u * j, db + 2u * j, idesc, (k | j) != 0 ? 1u : 0u);
                    else mma_tf32(acc, da + 2u * j, db + 2u * j, idesc, (k | j) != 0 ? 1u : 0u);
                }
                if (PAIR) mma_commit_pair(empty_bar + 8u * s);
                else mma_commit(empty_bar + 8u * s);
                dbg_mark(p, 3, (uint32_t)(k + 1));
                if (++s == stages) { s = 0; round++; }
            }
            if (ok) {
                if (PAIR) mma_commit_pair(acc_full + 8u * buf);
                else mma_commit(acc_full + 8u * buf);
                if (clk) p.clocks[local * 8 + 3] = clock64();
            }
        }
    } else if (warp >= 2) {
        // ---------------- epilogue
        const int quarter = warp & 3;
        const int row_in_tile = quarter * 32 + lane;
        const uint32_t lane_bits = (uint32_t)(quarter * 32) << 16;
        const bool issuer = threadIdx.x == 64;   // the thread that talks to the copy engine
        // swizzled position of this row's 16-byte chunk c inside a staging tile: chunk ^ (row & 7)
        const uint32_t row_base = (uint32_t)row_in_tile * 128u;
        const uint32_t row_phase = (uint32_t)row_in_tile & 7u;
        int local = 0, stage_buf = 0;
        bool ok = true;
        for (int t = worker; t < p.total_tiles && ok; t += n_workers, local++) {
            int mt, nt, bt, sp;
            tile_coords(t, mt, nt, bt, sp);
            if (PAIR) mt = 2 * mt + (int)rank;   // from here on: this CTA's 128-row block
            const int buf = local & 1;
            {
                uint32_t good = 1;
                if (lane == 0) good = mbar_wait(acc_full + 8u * buf, (uint32_t)((local >> 1) & 1), abandon, p.status, 24) ? 1u : 0u;
                good = __shfl_sync(0xffffffffu, good, 0);
                // the loop below synchronises the four epilogue warps with each other, so they must agree on
                // entering it: vote (every epilogue thread gets here, its wait being bounded)
                uint32_t all_good;
                asm volatile(
                    "{\n\t.reg .pred p, q;\n\t"
                    "setp.ne.u32 p, %1, 0;\n\t"
                    "bar.red.and.pred q, 2, 128, p;\n\t"
                    "selp.u32 %0, 1, 0, q;\n\t}"
                    : "=r"(all_good)
                    : "r"(good)
                    : "memory");
                if (!all_good) { ok = false; break; }
                while (!mbar_try_wait(acc_full + 8u * buf, (uint32_t)((local >> 1) & 1))) {}
            }
            tc_fence_after();
            const bool eclk = p.clocks != nullptr && blockIdx.x == 0 && local < kGpClockTiles && issuer;
            long long store_wait = 0;
            if (eclk) p.clocks[local * 8 + 4] = clock64();
            if (issuer) dbg_mark(p, 4, 1);
            const int64_t row = (int64_t)mt * kGpBlockM + row_in_tile;
            const bool row_ok = row < p.m;
            const int chunks = (p.bn + 31) >> 5;
            for (int c = 0; c < chunks; c++) {
                const int col0 = nt * p.bn + c * 32;
                if (col0 >= p.n) break;                       // uniform: nothing of this chunk is inside the matrix
                uint32_t v[32];
                tmem_load_32(tmem_base + lane_bits + (uint32_t)(buf * p.bn + c * 32), v);
                // addends: a per-column value is fetched once per chunk (lane j holds column col0 + j) and
                // handed round with shuffles; a per-element addend is this thread's own row, 128 contiguous bytes
#pragma unroll
                for (int which = 0; which < 2; which++) {
                    const int mode = which == 0 ? p.add1_mode : p.add2_mode;
                    if (mode == 0) continue;
                    const float* add = which == 0 ? p.add1 : p.add2;
                    const int64_t* st = which == 0 ? p.s1 : p.s2;
                    if (HALF) {
                        // f16 addends: converted on load
                        const __half* addh = (const __half*)add;
                        if (mode == 1) {
                            const int64_t col = col0 + lane;
                            const float mine = col < p.n ? __half2float(__ldg(addh + bt * st[0] + col * st[2])) : 0.f;
#pragma unroll
                            for (int j = 0; j < 32; j++) v[j] = __float_as_uint(__uint_as_float(v[j]) + __shfl_sync(0xffffffffu, mine, j));
                        } else if (mode == 4) {
                            const float mine = row_ok ? __half2float(__ldg(addh + bt * st[0] + row * st[1])) : 0.f;
#pragma unroll
                            for (int j = 0; j < 32; j++) v[j] = __float_as_uint(__uint_as_float(v[j]) + mine);
                        } else if (row_ok) {
                            const __half* src = addh + bt * st[0] + row * st[1] + col0;
                            if (col0 + 32 <= p.n && ((uintptr_t)src & 15) == 0) {
#pragma unroll
                                for (int q = 0; q < 4; q++) {
                                    const uint4 a8 = __ldg((const uint4*)src + q);
                                    const __half2* h2 = (const __half2*)&a8;
#pragma unroll
                                    for (int u = 0; u < 4; u++) {
                                        const float2 f = __half22float2(h2[u]);
                                        v[8 * q + 2 * u] = __float_as_uint(__uint_as_float(v[8 * q + 2 * u]) + f.x);
                                        v[8 * q + 2 * u + 1] = __float_as_uint(__uint_as_float(v[8 * q + 2 * u + 1]) + f.y);
                                    }
                                }
                            } else {
#pragma unroll
                                for (int j = 0; j < 32; j++)
                                    if (col0 + j < p.n) v[j] = __float_as_uint(__uint_as_float(v[j]) + __half2float(__ldg(src + j)));
                            }
                        }
                        continue;
                    }
                    if (mode == 1) {
                        const int64_t col = col0 + lane;
                        const float mine = col < p.n ? __ldg(add + bt * st[0] + col * st[2]) : 0.f;
#pragma unroll
                        for (int j = 0; j < 32; j++) v[j] = __float_as_uint(__uint_as_float(v[j]) + __shfl_sync(0xffffffffu, mine, j));
                    } else if (mode == 4) {
                        const float mine = row_ok ? __ldg(add + bt * st[0] + row * st[1]) : 0.f;
#pragma unroll
                        for (int j = 0; j < 32; j++) v[j] = __float_as_uint(__uint_as_float(v[j]) + mine);
                    } else if (row_ok) {
                        const float* src = add + bt * st[0] + row * st[1] + col0;
                        if (col0 + 32 <= p.n && ((uintptr_t)src & 15) == 0) {
#pragma unroll
                            for (int q = 0; q < 8; q++) {
                                const float4 a4 = __ldg((const float4*)src + q);
                                v[4 * q] = __float_as_uint(__uint_as_float(v[4 * q]) + a4.x);
                                v[4 * q + 1] = __float_as_uint(__uint_as_float(v[4 * q + 1]) + a4.y);
                                v[4 * q + 2] = __float_as_uint(__uint_as_float(v[4 * q + 2]) + a4.z);
                                v[4 * q + 3] = __float_as_uint(__uint_as_float(v[4 * q + 3]) + a4.w);
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; j++)
                                if (col0 + j < p.n) v[j] = __float_as_uint(__uint_as_float(v[j]) + __ldg(src + j));
                        }
                    }
                }
                if (p.act == (int)Activation::Relu) {
#pragma unroll
                    for (int j = 0; j < 32; j++) v[j] = __float_as_uint(fmaxf(__uint_as_float(v[j]), 0.f));
                } else if (p.act == (int)Activation::Gelu) {
#pragma unroll
                    for (int j = 0; j < 32; j++) v[j] = __float_as_uint(gelu_erf_tensor_core(__uint_as_float(v[j])));
                }
                // the staging tile about to be written was handed to the copy engine two chunks ago
                if (issuer) {
                    const long long t0 = eclk ? clock64() : 0;
                    asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                    if (eclk) store_wait += clock64() - t0;
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (HALF && p.out_half) {
                    // f16 output: rows of 32 halves = 64 bytes, plain row-major (the store map has no swizzle)
                    const uint32_t stile = staging_base + (uint32_t)stage_buf * kGpStageTileBytes + (uint32_t)row_in_tile * 64u;
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        uint32_t h[4];
#pragma unroll
                        for (int u = 0; u < 4; u++) {
                            const __half2 pair = __floats2half2_rn(__uint_as_float(v[8 * q + 2 * u]), __uint_as_float(v[8 * q + 2 * u + 1]));
                            h[u] = *(const uint32_t*)&pair;
                        }
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(stile + (uint32_t)q * 16u), "r"(h[0]), "r"(h[1]),
                                     "r"(h[2]), "r"(h[3])
                                     : "memory");
                    }
                } else {
                    const uint32_t stile = staging_base + (uint32_t)stage_buf * kGpStageTileBytes + row_base;
#pragma unroll
                    for (int q = 0; q < 8; q++)
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(stile + (((uint32_t)q ^ row_phase) << 4)),
                                     "r"(v[4 * q]), "r"(v[4 * q + 1]), "r"(v[4 * q + 2]), "r"(v[4 * q + 3])
                                     : "memory");
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (issuer) {
                    tma_store_3d(&map_c, staging_base + (uint32_t)stage_buf * kGpStageTileBytes, col0, mt * kGpBlockM, bt * p.splits + sp);
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    dbg_mark(p, 5, (uint32_t)(c + 1));
                }
                stage_buf ^= 1;
            }
            if (eclk) p.clocks[local * 8 + 5] = clock64(), p.clocks[local * 8 + 6] = store_wait;
            // every tcgen05.ld of this accumulator has completed (tmem_load_32 waits): the MMA thread may reuse it
            tc_fence_before();
            if (PAIR) mbar_arrive_cluster(map_to_cta(acc_empty + 8u * buf, 0));
            else mbar_arrive_local(acc_empty + 8u * buf);
        }
        if (issuer) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // shared memory must outlive the stores
        if (issuer) dbg_mark(p, 6, 1);
    }

    tc_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync_all();   // neither CTA leaves (or frees tensor memory) while the other may still address it
    if (warp == 0) {
        if (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
        else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
    }
}

struct GemmPersistentLaunch {
    CUtensorMap map_a, map_b, map_c;
    GemmPersistentParams p;
    dim3 grid;
    int smem_bytes;
    bool half;
    bool pair;   // CTA pairs (clusters of two, cta_group::2)
};

// 0 absent, 1 one value per column (row stride 0), 2 a value per element with contiguous rows, 4 one value per
// row (column stride 0), 3 anything else
int classify_addend(const float* ptr, const int64_t* st) {
    if (ptr == nullptr) return 0;
    if (st[1] == 0) return 1;
    if (st[2] == 1) return 2;
    if (st[2] == 0) return 4;
    return 3;
}

}  // namespace

// Column blocks of equal width: n = 320 is two blocks of 160, not 256 + 64 with three quarters of the second empty.
int gemm_persistent_bn(int64_t n) {
    if (const char* e = getenv("KN_GEMM_BN")) {   // (measuring: a fixed block width, a multiple of 32)
        const int v = atoi(e);
        if (v >= 32 && v <= 256 && v % 32 == 0 && n >= v) return v;
    }
    const int64_t blocks = (n + 255) / 256;
    // (several blocks: a multiple of 32, the width of an epilogue chunk, so that no chunk reaches into the
    // next block's columns; a single block is clipped by the store's tensor bounds)
    const int64_t unit = blocks > 1 ? 32 : 16;
    return (int)std::min<int64_t>(((n + blocks - 1) / blocks + unit - 1) / unit * unit, 256);
}

std::shared_ptr<void> gemm_persistent_prepare(const GemmParams& g, uint32_t* status_word, int splits, int k_iters_slice,
                                              uint32_t* trace_words) {
    if (g.batch < 1 || g.m < 1 || g.n < 16 || g.k < 1 || splits < 1) return nullptr;
    const bool split = splits > 1;
    const bool half = g.half != 0;
    const int64_t align = half ? 8 : 4;            // elements per 16 bytes
    const int block_k = half ? 64 : 32;
    // dense row-major C whose rows start on 16-byte boundaries (split K: the partial sums [batch][slice][m][n],
    // which the reduction kernel turns into C; addends and activation are applied there)
    if (split) {
        if (g.n % 4 != 0 || ((uintptr_t)g.scratch & 15) != 0 || g.scratch == nullptr) return nullptr;
    } else if (g.sc[2] != 1 || g.sc[1] % align != 0 || (g.batch > 1 && g.sc[0] % align != 0) || ((uintptr_t)g.c & 15) != 0) {
        return nullptr;
    }
    const int m1 = split ? 0 : classify_addend(g.add1, g.s1), m2 = split ? 0 : classify_addend(g.add2, g.s2);
    if (m1 == 3 || m2 == 3) return nullptr;
    auto l = std::make_shared<GemmPersistentLaunch>();
    GemmPersistentParams& p = l->p;
    memset(&p, 0, sizeof(p));
    p.bn = gemm_persistent_bn(g.n);
    p.k_iters = (int)((g.k + block_k - 1) / block_k);
    p.out_half = half && !split ? 1 : 0;
    l->half = half;
    p.n_tiles = (int)((g.n + p.bn - 1) / p.bn);
    // CTA pairs: at least one 256-row tile per pair of SMs, and a reduction long enough
    // for the mainloop to matter (measured, f32: 11 % faster at 24 K blocks and more, even at 16, 8 to 17 % slower at
    // 2 to 10, where a tile is mostly epilogue and the pair's hand-offs cost more than the operand traffic they save).
    // KN_GEMM_PAIR=0 in the environment switches pairs off, KN_GEMM_PAIR=1 drops the K condition (A/B measurements).
    // (no K slices; the A operand may be a head split or merge read in place, 42.3 -> 38.5 us on the BERT output
    // projection; with convolution windows as the A operand pairs measured no faster, 127.4 against 126.3 us, and a B
    // operand read in place would need its box halved: those stay on one CTA per tile)
    bool pair = !split && g.conv_operand == 0 && !g.b4.enabled && p.bn % 32 == 0 && p.bn >= 64 && g.m >= 256 &&
                ((g.m + 255) / 256) * p.n_tiles * g.batch >= 74;
    const char* pair_env = getenv("KN_GEMM_PAIR");
    if (pair_env && atoi(pair_env) == 0) pair = false;
    if (!pair_env && p.k_iters < 20) pair = false;
    l->pair = pair;
    p.m_tiles = (int)((g.m + (pair ? 2 : 1) * kGpBlockM - 1) / ((pair ? 2 : 1) * kGpBlockM));
    p.batch = (int)g.batch;
    p.splits = splits;
    p.k_iters_slice = split ? k_iters_slice : p.k_iters;
    if ((int64_t)(splits - 1) * p.k_iters_slice >= p.k_iters) return nullptr;   // an empty slice
    const int64_t total = (int64_t)p.m_tiles * p.n_tiles * g.batch * splits;
    if (total > (1 << 30)) return nullptr;
    p.total_tiles = (int)total;
    p.m = g.m;
    p.n = g.n;
    p.add1 = g.add1;
    p.add2 = g.add2;
    for (int i = 0; i < 3; i++) {
        p.s1[i] = g.s1[i];
        p.s2[i] = g.s2[i];
    }
    p.add1_mode = m1;
    p.add2_mode = m2;
    p.act = split ? 0 : g.act;
    p.status = status_word;
    p.dbg = (volatile uint32_t*)trace_words;
    // KN_GEMM_CLOCKS=1 in the environment: CTA 0 stamps clock64 per tile (MMA thread: tile reached, accumulator free,
    // first K block landed, all MMAs issued; copy-engine thread of the epilogue: accumulator ready, tile stored, cycles
    // spent waiting for staging tiles) and the table of the last launch is printed when the process exits.
    if (getenv("KN_GEMM_CLOCKS")) {
        static long long* table = nullptr;
        if (!table && cudaHostAlloc((void**)&table, (size_t)kGpClockTiles * 64, cudaHostAllocMapped) == cudaSuccess) {
            atexit([] {
                const long long* d = table;
                fprintf(stderr, "gemm_persistent_kernel, CTA 0, SM clock cycles since the MMA thread reached the tile\n"
                                "tile  accumulator_free  first_block_landed  mmas_issued  | accumulator_ready  tile_stored  (staging waits)  | period\n");
                for (int i = 0; i < kGpClockTiles && d[i * 8 + 3]; i++)
                    fprintf(stderr, "%4d  %16lld  %18lld  %11lld  | %17lld  %11lld  %15lld  | %6lld\n", i, d[i * 8 + 1] - d[i * 8], d[i * 8 + 2] - d[i * 8],
                            d[i * 8 + 3] - d[i * 8], d[i * 8 + 4] - d[i * 8], d[i * 8 + 5] - d[i * 8], d[i * 8 + 6], i ? d[i * 8] - d[(i - 1) * 8] : 0);
            });
        }
        if (table) memset(table, 0, (size_t)kGpClockTiles * 64);
        p.clocks = table;
    }
    const int stage_bytes = kGpATileBytes + (pair ? p.bn / 2 : p.bn) * 128;
    const int fixed = 1024 + 2 * kGpStageTileBytes + 16 * 8 + 64 + 64;
    p.stages = std::max(2, std::min(6, (227 * 1024 - fixed) / stage_bytes));
    l->smem_bytes = fixed + p.stages * stage_bytes;
    p.a_batch = (g.batch > 1 && g.sa[0] == 0) ? 0 : 1;
    int64_t adims[3] = {g.k, g.m, p.a_batch ? g.batch : 1}, astr[3] = {1, g.sa[1], p.a_batch ? g.sa[0] : align};
    int abox[3] = {block_k, kGpBlockM, 1};
    p.b_batch = (g.batch > 1 && g.sb[0] == 0) ? 0 : 1;
    int64_t bdims[3] = {g.k, g.n, p.b_batch ? g.batch : 1}, bstr[3] = {1, g.sb[2], p.b_batch ? g.sb[0] : align};
    int bbox[3] = {block_k, pair ? p.bn / 2 : p.bn, 1};
    // the implicit convolution operand: a 4-D map of the image tensor (channel, x, y, image) whose box is one K
    // block of channels by whole output rows
    int64_t idims[4] = {g.conv_c, g.conv_w, g.conv_h, g.batch}, istr[4] = {1, g.conv_strides[2], g.conv_strides[1], g.conv_strides[0]};
    int ibox[4] = {32, 1, 1, 1};
    if (g.conv_operand != 0) {
        const int rows = g.conv_operand == 1 ? kGpBlockM : p.bn;
        if (half || g.conv_c % 32 != 0 || g.conv_ow < 1 || g.conv_ow > 256 || rows % g.conv_ow != 0 || g.conv_r < 1 || g.conv_s < 1 ||
            g.k != (int64_t)g.conv_r * g.conv_s * g.conv_c)
            return nullptr;
        ibox[1] = g.conv_ow;
        ibox[2] = rows / g.conv_ow;
        p.conv_operand = g.conv_operand;
        p.conv_cblocks = g.conv_c / 32;
        p.conv_s = g.conv_s;
        p.conv_pad_y = g.conv_pad_y;
        p.conv_pad_x = g.conv_pad_x;
        p.conv_ow = g.conv_ow;
    }
    // 4-D operands: the box is one K block by the tile's rows inside one (x, y) entry
    auto operand_4d = [&](const GemmOperand4D& o, const void* base, int rows, int64_t matrix_rows, int32_t* kd_shift, int32_t* rd, int32_t* bi,
                          CUtensorMap* map) {
        if (!o.enabled) return true;
        if (o.kd < 1 || o.rd < 1 || o.bi < 1 || o.strides[0] != 1 || g.conv_operand != 0) return false;
        int shift = 0;
        if (o.kd != g.k) {   // the K offset is split: whole K blocks inside one entry, by a shift
            if (o.kd % block_k != 0 || (o.kd & (o.kd - 1)) != 0) return false;
            while ((1 << shift) < o.kd) shift++;
        }
        // a tile's rows lie inside one entry: an entry's rows are a multiple of the tile's, or the matrix is one entry
        // tall (then rows past its end are past the tensor's extent: zero fill)
        if (o.rd % rows != 0 && o.rd < matrix_rows) return false;
        int box[4] = {block_k, rows, 1, 1};
        *map = half ? tc_make_map_f16(base, 4, o.dims, o.strides, box, true) : tc_make_map(base, 4, o.dims, o.strides, box, true);
        *kd_shift = shift;
        *rd = o.rd;
        *bi = o.bi;
        return true;
    };
    if (!operand_4d(g.a4, g.a, kGpBlockM, g.m, &p.a4_kd_shift, &p.a4_rd, &p.a4_bi, &l->map_a)) return nullptr;
    if (!operand_4d(g.b4, g.b, p.bn, g.n, &p.b4_kd_shift, &p.b4_rd, &p.b4_bi, &l->map_b)) return nullptr;
    if (g.a4.enabled && g.b4.enabled) {
    } else if (g.a4.enabled) {
        l->map_b = half ? tc_make_map_f16(g.b, 3, bdims, bstr, bbox, true) : tc_make_map(g.b, 3, bdims, bstr, bbox, true);
    } else if (g.b4.enabled) {
        l->map_a = half ? tc_make_map_f16(g.a, 3, adims, astr, abox, true) : tc_make_map(g.a, 3, adims, astr, abox, true);
    } else if (half) {
        l->map_a = tc_make_map_f16(g.a, 3, adims, astr, abox, true);
        l->map_b = tc_make_map_f16(g.b, 3, bdims, bstr, bbox, true);
    } else {
        l->map_a = g.conv_operand == 1 ? tc_make_map(g.a, 4, idims, istr, ibox, true) : tc_make_map(g.a, 3, adims, astr, abox, true);
        l->map_b = g.conv_operand == 2 ? tc_make_map(g.b, 4, idims, istr, ibox, true) : tc_make_map(g.b, 3, bdims, bstr, bbox, true);
    }
    int64_t cdims[3] = {g.n, g.m, g.batch * splits}, cstr[3] = {1, split ? g.n : g.sc[1], split ? g.m * g.n : g.sc[0]};
    int cbox[3] = {32, kGpBlockM, 1};
    if (p.out_half) l->map_c = tc_make_map_f16(g.c, 3, cdims, cstr, cbox, false);
    else l->map_c = tc_make_store_map(split ? g.scratch : g.c, 3, cdims, cstr, cbox);
    l->grid = pair ? dim3(2u * (unsigned)std::min<int64_t>(total, 74), 1, 1) : dim3((unsigned)std::min<int64_t>(total, 148), 1, 1);
    return l;
}

int gemm_persistent_launch(const void* launch, cudaStream_t stream) {
    const GemmPersistentLaunch& l = *(const GemmPersistentLaunch*)launch;
    static std::mutex mu;
    static bool done[64] = {false};
    int device = 0;
    cudaGetDevice(&device);
    {
        std::lock_guard<std::mutex> lock(mu);
        if (device >= 0 && device < 64 && !done[device]) {
            const void* variants[] = {(const void*)gemm_persistent_kernel<false, false>, (const void*)gemm_persistent_kernel<true, false>,
                                      (const void*)gemm_persistent_kernel<false, true>, (const void*)gemm_persistent_kernel<true, true>};
            for (const void* v : variants) {
                cudaError_t e = cudaFuncSetAttribute(v, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
                if (e != cudaSuccess) return (int)e;
            }
            done[device] = true;
        }
    }
    if (l.pair) {
        // clusters of two CTAs, still with the programmatic edge to the previous kernel
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = l.grid;
        cfg.blockDim = dim3(kGpThreads);
        cfg.dynamicSmemBytes = (size_t)l.smem_bytes;
        cfg.stream = stream;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        attr[1].id = cudaLaunchAttributeClusterDimension;
        attr[1].val.clusterDim.x = 2;
        attr[1].val.clusterDim.y = 1;
        attr[1].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 2;
        if (l.half) return (int)cudaLaunchKernelEx(&cfg, gemm_persistent_kernel<true, true>, l.map_a, l.map_b, l.map_c, l.p);
        return (int)cudaLaunchKernelEx(&cfg, gemm_persistent_kernel<false, true>, l.map_a, l.map_b, l.map_c, l.p);
    }
    if (l.half) launch_pdl(gemm_persistent_kernel<true, false>, dim3(l.grid), dim3(kGpThreads), (size_t)(l.smem_bytes), stream, l.map_a, l.map_b, l.map_c, l.p);
    else launch_pdl(gemm_persistent_kernel<false, false>, dim3(l.grid), dim3(kGpThreads), (size_t)(l.smem_bytes), stream, l.map_a, l.map_b, l.map_c, l.p);
    return (int)cudaGetLastError();
}

}  // namespace kn
