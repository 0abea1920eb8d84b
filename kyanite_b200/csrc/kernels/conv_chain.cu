// A run of 3x3 stride-1 same-padding convolutions (a residual tower) as ONE kernel for sm_100a.
//
// A 3x3 convolution of an image reads that image only, so a CTA that owns a few whole images can run
// every layer of the run back to back without ever leaving its SM: the activations live in shared
// memory (as the B operand of the next layer's MMAs), the skip connection of a residual block lives in
// tensor memory next to the accumulator, and per layer only the filter streams in from L2 through a
// small ring (one request per filter tap: up to four 16 KB tiles, stored by the planner in the swizzled
// byte order of shared memory so a linear bulk copy delivers them).  Compared with one launch per layer
// this removes, per layer, the launch, the pipeline fill, the activation round trip through L2 and the
// output store.
//
// Accumulator orientation: D[output channel = TMEM lane][padded position = column].
//   A operand  filter tile [128 output channels x 32 input channels], K-major, 128-byte swizzle, copied
//              with `cp.async.bulk` from a tile array the planner lays out tap by tap
//   B operand  the activation buffer: per 32-channel block, one 128-byte row per padded position, same
//              swizzle.  The images are stored as one tall zero-padded image (ChainGeometry, tc.h), so
//              filter tap (r, s) is the same operand started `(r-1) * wp + (s-1)` rows further on.  Such a
//              start is 128-byte but not 1024-byte aligned.  The tensor core resolves the swizzle from the
//              absolute shared-memory address (16-byte chunk index XOR address bits 7..9), and the buffer's
//              pattern is anchored at a 1024-byte boundary, so the descriptor's base-offset field stays 0
//              (measured: a non-zero base offset permutes the channels).
//
// Warp roles (64 + 128 E threads): warp 0 lane 0 streams filter tiles; warp 1 lane 0 issues the MMAs of a layer
// once its input is complete; the other 4 E warps are the epilogue (E warps per TMEM lane quarter, taking the
// 16-column chunks of the accumulator in turn; E = 3 when the chunk count divides by three, as the 9 chunks of
// two 8x8 boards do, else 2): accumulator + bias (+ held skip tensor) -> ReLU -> written back as the
// next layer's operand (rounded to TF32, zeros at padding positions) and, if a later layer adds it,
// into the held-tensor columns of TMEM in full f32; a layer flagged to store writes its result to global
// memory.  The last layer may be a pointwise (1x1) layer that computes several convolutions of the last
// 3x3 result at once, their output channels side by side in the accumulator's lanes ("heads": each with
// its own output tensor and activation), so the tower's result need not leave the SM at all.
//
// Every mbarrier wait is bounded; on expiry the executor's status word is raised, all roles leave, TMEM is
// freed and the kernel returns.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstring>
#include <memory>
#include <mutex>

#include "../tc.h"
#include "tc_host.h"
#include "tc_ptx.cuh"

namespace kn {

namespace {

using namespace tcp;

constexpr int kChainThreadsMin = 320;    // every variant has at least this many threads (set-up loops rely on >= 256)
constexpr int kTileBytes = 128 * 128;   // one filter tile: 128 rows of 128 bytes

struct ChainKernelParams {
    const float* in;
    float* out;
    const float* bias;
    const float* tiles;
    int64_t s_in[4], s_out[4];
    int32_t n_img, c_in, k, h, w;
    int32_t n_layers, per_cta, gx, gy, wp, q_first, r_first, n_mma, rows_alloc, slots, tmem_cols, c_blocks_max;
    int32_t total_tiles;
    int32_t group;   // filter tiles per request and per ring slot
    long long* trace; // KN_CHAIN_TRACE only: per layer 8 clock64 stamps of CTA 0, in pinned host memory
    uint8_t flags[kMaxChainLayers];
    uint8_t c_blocks[kMaxChainLayers];
    uint32_t* status;
    int32_t n_heads;
    int32_t head_begin[kMaxChainHeads + 1];
    float* head_out[kMaxChainHeads];
    int64_t head_s_out[kMaxChainHeads][4];
    uint8_t head_relu[kMaxChainHeads];
};

__device__ __forceinline__ void tmem_store_16(uint32_t taddr, const uint32_t (&v)[16]) {   // caller waits (tcgen05.wait::st)
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
          "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
        : "memory");
}

__device__ __forceinline__ void tmem_load_16_nowait(uint32_t taddr, uint32_t (&v)[16]) {   // caller waits (tcgen05.wait::ld)
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_store_8(uint32_t taddr, const uint32_t (&v)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
                 : "memory");
}
__device__ __forceinline__ void tmem_load_8_nowait(uint32_t taddr, uint32_t (&v)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                 : "r"(taddr)
                 : "memory");
}
template <int CW> __device__ __forceinline__ void tmem_store_chunk(uint32_t taddr, const uint32_t (&v)[CW]) {
    if constexpr (CW == 16) tmem_store_16(taddr, v); else tmem_store_8(taddr, v);
}
template <int CW> __device__ __forceinline__ void tmem_load_chunk_nowait(uint32_t taddr, uint32_t (&v)[CW]) {
    if constexpr (CW == 16) tmem_load_16_nowait(taddr, v); else tmem_load_8_nowait(taddr, v);
}

// Suspend-time hint of the kernel's mbarrier waits: a waiting thread is woken when the phase completes, so the hint
// only bounds how long it sleeps between two looks at the abandon flag.
constexpr uint32_t kSleepNs = 20000u;

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// E: epilogue warps per TMEM lane quarter; CW: accumulator columns per epilogue chunk (16 or 8); TRACE: whether the
// first CTA stamps its phases
template <int E, int CW, bool TRACE>
__global__ void __launch_bounds__(64 + 128 * E, 1)
conv_chain_kernel(const __grid_constant__ CUtensorMap map_tiles, const __grid_constant__ ChainKernelParams p) {
    constexpr int kChainThreads = 64 + 128 * E;
    constexpr int kEpilogueThreads = 128 * E;
    static_assert(kChainThreads >= kChainThreadsMin, "set-up loops assume at least 320 threads");
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t block_bytes = (uint32_t)p.rows_alloc * 128u;                 // one 32-channel block of activations
    const uint32_t act_bytes = (uint32_t)p.c_blocks_max * block_bytes;
    const uint32_t ring_base = base + act_bytes;
    const uint32_t slot_bytes = (uint32_t)p.group * kTileBytes;
    const uint32_t bar_base = ring_base + (uint32_t)p.slots * slot_bytes;
    const uint32_t full_bar = bar_base, empty_bar = bar_base + 8u * p.slots;
    const uint32_t accum_bar = bar_base + 16u * p.slots, act_bar = accum_bar + 8u;
    const uint32_t slot_addr = act_bar + 8u;
    volatile uint32_t* tmem_slot = (volatile uint32_t*)(gen_base + (slot_addr - base));
    volatile int* abandon = (volatile int*)(gen_base + (slot_addr + 4u - base));
    uint32_t* colinfo = (uint32_t*)(gen_base + (slot_addr + 8u - base));         // 256 entries
    uint32_t* realmask = colinfo + 256;                                          // 32 entries: per CW-column chunk, which columns are real pixels
    const uint32_t dummy_rows = slot_addr + 8u + 1024u + 128u + 24u;             // (16-byte aligned) 128 bytes nobody reads: where the stores of padding positions go
    volatile int* epilogue_go = (volatile int*)(realmask + 32);                  // 2 entries: the accumulator poller's verdict, per layer parity

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.slots; s++) {
            mbar_init(full_bar + 8u * s, 1);
            mbar_init(empty_bar + 8u * s, 1);
        }
        mbar_init(accum_bar, 1);
        mbar_init(act_bar, kEpilogueThreads / 32);   // one arrival per epilogue warp
        *abandon = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // the activation buffer starts as zeros: padding positions and guard rows are never written with
    // anything else
    {
        uint4* z = (uint4*)gen_base;
        const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
        for (uint32_t i = threadIdx.x; i < act_bytes / 16u; i += kChainThreads) z[i] = zero;
    }
    // column -> pixel table: bit 31 real pixel, bits 16..23 image within the CTA, 8..15 y, 0..7 x
    if (threadIdx.x < 256) {
        const int n = threadIdx.x;
        uint32_t info = 0;
        if (n < p.n_mma) {
            const int q = n + p.q_first;
            const int row = q / p.wp, col = q - row * p.wp;
            const int iy = row / (p.h + 1), ry = row - iy * (p.h + 1);
            const int ix = col / (p.w + 1), cx = col - ix * (p.w + 1);
            const int img = iy * p.gx + ix;
            if (cx != 0 && ry != 0 && iy < p.gy && (int64_t)blockIdx.x * p.per_cta + img < p.n_img)
                info = 0x80000000u | ((uint32_t)img << 16) | ((uint32_t)(ry - 1) << 8) | (uint32_t)(cx - 1);
        }
        colinfo[n] = info;
    }
    __syncthreads();
    if (threadIdx.x >= 64 && threadIdx.x < 64 + 256 / CW) {
        const int c = threadIdx.x - 64;
        uint32_t m = 0;
        for (int j = 0; j < CW; j++) m |= (colinfo[c * CW + j] >> 31) << j;
        realmask[c] = m;
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_addr), "r"((uint32_t)p.tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_acc = *tmem_slot;
    const uint32_t tmem_held = tmem_acc + (uint32_t)p.n_mma;      // n_mma is a multiple of 16

    if (warp == 0 && lane == 0) {
        // ---------------- filter producer: tiles are consumed in the order they are stored; the filter
        // is a constant of the plan, so nothing here waits for the previous kernel
        // Within a layer the tiles may be consumed in any order (they all accumulate into the same
        // tile), so every CTA starts at a different one: at any moment the SMs then pull different
        // lines from L2 instead of all hammering the slice that holds the current tile.
        // (ring position and indices are advanced by hand: integer division by a run-time value costs
        // tens of cycles, and this loop runs once per request)
        int layer_base = 0, slot = 0, round = 0;
        bool ok = true;
        for (int l = 0; l < p.n_layers && ok; l++) {
            const int n = ((p.flags[l] & kChainFlagPointwise) ? 1 : 9) * p.c_blocks[l];
            const int g = n % p.group == 0 ? p.group : 1;      // tiles per request
            const int groups = n / g;
            int idx = (int)((blockIdx.x * 5u) % (uint32_t)groups);
            for (int i = 0; i < groups; i++) {
                if (round > 0) {
                    if (!mbar_wait(empty_bar + 8u * slot, (uint32_t)((round & 1) ^ 1), abandon, p.status, 11, kWaitCycles, kSleepNs)) { ok = false; break; }
                }
                const uint32_t bar = full_bar + 8u * slot;
                mbar_expect_tx(bar, (uint32_t)g * kTileBytes);
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"(ring_base + (uint32_t)slot * slot_bytes), "l"(p.tiles + (size_t)(layer_base + idx * g) * (kTileBytes / 4)),
                               "r"((uint32_t)g * kTileBytes), "r"(bar)
                             : "memory");
                if (++idx == groups) idx = 0;
                if (++slot == p.slots) { slot = 0; round++; }
            }
            layer_base += n;
        }
    } else if (warp == 1 && lane == 0) {
        // ---------------- MMA issuer
        const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(p.n_mma >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
        int slot = 0, round = 0;
        bool ok = true;
        const bool trace = TRACE && blockIdx.x == 0;
        for (int l = 0; l < p.n_layers && ok; l++) {
            long long t0 = 0, full_wait = 0;
            if (trace) t0 = clock64();
            // the layer's input is complete in shared memory and the accumulator has been read out
            ok = mbar_wait(act_bar, (uint32_t)(l & 1), abandon, p.status, 12, kWaitCycles, kSleepNs);
            if (!ok) break;
            if (trace) p.trace[l * 8 + 0] = t0, p.trace[l * 8 + 1] = clock64();
            tc_fence_after();
            // The next kernel of the stream may be scheduled once every CTA is in its last layer: early enough
            // to hide that kernel's launch and set-up, late enough that its CTAs do not sit on this SM (blocked
            // in griddepcontrol.wait) for the whole run.
            if (l == p.n_layers - 1) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
            const int cbl = p.c_blocks[l];
            uint32_t accumulate = 0;
            const bool pointwise = (p.flags[l] & kChainFlagPointwise) != 0;
            const int n = (pointwise ? 1 : 9) * cbl;
            const int g = n % p.group == 0 ? p.group : 1;
            const int groups = n / g;
            // the producer's order: start at group (blockIdx.x * 5) % groups, wrap around
            int tile = (int)((blockIdx.x * 5u) % (uint32_t)groups) * g;
            int tap = tile / cbl, cb = tile - tap * cbl;
            if (pointwise) tap = 4;     // the centre tap: the operand starts at the pixel itself
            for (int i = 0; i < groups && ok; i++) {
                long long tw = 0;
                if (trace) tw = clock64();
                ok = mbar_wait(full_bar + 8u * slot, (uint32_t)(round & 1), abandon, p.status, 13, kWaitCycles, kSleepNs);
                if (!ok) break;
                if (trace) full_wait += clock64() - tw;
                tc_fence_after();
                for (int u = 0; u < g; u++) {
                    const int r = tap >= 6 ? 2 : (tap >= 3 ? 1 : 0), s = tap - 3 * r;
                    const uint32_t row0 = (uint32_t)(p.r_first + (r - 1) * p.wp + (s - 1));
                    const uint64_t da = smem_desc_sw128(ring_base + (uint32_t)slot * slot_bytes + (uint32_t)u * kTileBytes);
                    const uint64_t db = smem_desc_sw128(base + (uint32_t)cb * block_bytes + row0 * 128u);
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        mma_tf32(tmem_acc, da + 2u * j, db + 2u * j, idesc, accumulate);
                        accumulate = 1;
                    }
                    if (++cb == cbl) {
                        cb = 0;
                        if (!pointwise && ++tap == 9) tap = 0;
                    }
                }
                mma_commit(empty_bar + 8u * slot);
                if (++slot == p.slots) { slot = 0; round++; }
            }
            if (ok) mma_commit(accum_bar);
            if (trace) p.trace[l * 8 + 2] = clock64(), p.trace[l * 8 + 3] = full_wait;
        }
    } else if (warp >= 2) {
        // ---------------- epilogue: thread <-> accumulator lane <-> channel; the two warps of a lane
        // quarter take alternate 16-column chunks
        const int quarter = warp & 3;
        const int half = (warp - 2) >> 2;      // which of the quarter's E warps this is: it takes chunks half, half + E, ...
        const int ch = quarter * 32 + lane;
        const uint32_t lane_bits = (uint32_t)(quarter * 32) << 16;
        const int64_t img0 = (int64_t)blockIdx.x * p.per_cta;
        const bool has_block = (ch >> 5) < p.c_blocks_max;     // narrower layers: no operand rows for these channels
        const uint32_t chunk = (uint32_t)(ch >> 2) & 7u;
        // this channel's 4 bytes inside a 128-byte row of its 32-channel block, before the swizzle
        const int chunks = p.n_mma / CW;      // n_mma is a multiple of 16
        // Output column n is stored in row r_first + n of the channel's block; r_first is a multiple of 8, so
        // the swizzle phase of a row (row & 7) is the column's n & 7, known at compile time inside the
        // unrolled loops: the eight swizzled chunk offsets are computed once.
        uint32_t sw[8];
#pragma unroll
        for (int i = 0; i < 8; i++) sw[i] = (chunk ^ (uint32_t)i) << 4;
        const uint32_t block_rows = base + (uint32_t)(ch >> 5) * block_bytes + (uint32_t)p.r_first * 128u;   // this quarter's channel block, row of column 0
        const uint32_t my_rows = base + (uint32_t)(ch >> 5) * block_bytes + (uint32_t)(ch & 3) * 4u + (uint32_t)p.r_first * 128u;
        // round to TF32 (nearest, ties away from zero) with integer arithmetic: the tensor core ignores
        // the low 13 mantissa bits, so adding half an ulp of TF32 to the magnitude is all it takes
        auto store_operand = [&](uint32_t chunk_rows, int j, float v) {
            uint32_t u = __float_as_uint(v);
            if ((u & 0x7F800000u) != 0x7F800000u) u += 0x1000u;
            asm volatile("st.shared.b32 [%0], %1;" ::"r"(chunk_rows + sw[j & 7] + (uint32_t)j * 128u), "r"(u) : "memory");
        };
        // the head this thread's channel belongs to in the pointwise last layer
        int head = -1;
        for (int i = 0; i < p.n_heads; i++)
            if (ch >= p.head_begin[i] && ch < p.head_begin[i + 1]) head = i;
        // layer 0's input: from global memory into the operand layout and the held-tensor columns
        asm volatile("griddepcontrol.wait;" ::: "memory");
        for (int c = half; c < chunks; c += E) {
            uint32_t v[CW];
#pragma unroll
            for (int j = 0; j < CW; j++) {
                const uint32_t info = colinfo[c * CW + j];
                float x = 0.f;
                if ((info >> 31) && ch < p.c_in)
                    x = p.in[(img0 + ((info >> 16) & 0xFF)) * p.s_in[0] + (int64_t)ch * p.s_in[1] + (int64_t)((info >> 8) & 0xFF) * p.s_in[2] +
                             (int64_t)(info & 0xFF) * p.s_in[3]];
                v[j] = __float_as_uint(x);
                if (has_block) store_operand(my_rows + (uint32_t)c * (CW * 128u), j, x);
            }
            tmem_store_chunk<CW>(tmem_held + lane_bits + (uint32_t)(c * CW), v);
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> tensor-core reads
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(act_bar);

        for (int l = 0; l < p.n_layers; l++) {
            const uint32_t flags = p.flags[l];
            const bool last = l == p.n_layers - 1;
            const bool heads = last && p.n_heads > 0;
            const bool add_held = (flags & kChainFlagAddHeld) != 0;
            const bool hold = (flags & kChainFlagHold) != 0 && !last;
            // where this thread's channel goes in global memory, if anywhere
            bool relu = (flags & kChainFlagRelu) != 0, valid = ch < p.k, to_global = (flags & kChainFlagStore) != 0;
            float* o_ptr = p.out + (int64_t)ch * p.s_out[1];
            int64_t o_s0 = p.s_out[0], o_s2 = p.s_out[2], o_s3 = p.s_out[3];
            if (heads) {
                valid = to_global = head >= 0;
                if (valid) {
                    relu = p.head_relu[head] != 0;
                    o_ptr = p.head_out[head] + (int64_t)(ch - p.head_begin[head]) * p.head_s_out[head][1];
                    o_s0 = p.head_s_out[head][0], o_s2 = p.head_s_out[head][2], o_s3 = p.head_s_out[head][3];
                }
            }
            const float bias = valid ? p.bias[l * 128 + ch] : 0.f;
            // ONE thread of the CTA polls, with a long suspend hint; the other epilogue threads sleep in a hardware
            // barrier.  During the mainloop the shared-memory data pipe is the busiest unit of the SM (the tensor core
            // reads both operands through it and the copy engine writes the filters through it), and every poll of
            // an mbarrier is a shared-memory access: a dozen polling warps took a measurable share of it.  The
            // poller publishes its verdict (go on / abandon) in a word per layer parity, so that all threads take
            // the same branch and none is left waiting in the barrier.
            const bool trace = TRACE && blockIdx.x == 0 && warp == 2 && lane == 0;
            if (trace) p.trace[l * 8 + 4] = clock64();
            {
                if (warp == 2 && lane == 0) {
                    int go = 1;
                    const long long start = clock64();
                    while (!mbar_try_wait_hint(accum_bar, (uint32_t)(l & 1), kSleepNs)) {
                        if (*abandon) { go = 0; break; }
                        if (clock64() - start > kWaitCycles) {
                            *abandon = 1;
                            atomicMax(p.status, 14u);
                            go = 0;
                            break;
                        }
                    }
                    epilogue_go[l & 1] = go;
                }
                asm volatile("bar.sync 1, %0;" ::"n"(kEpilogueThreads) : "memory");
                if (!epilogue_go[l & 1]) break;
            }
            tc_fence_after();
            if (trace) p.trace[l * 8 + 5] = clock64();
            {
                // Software pipeline over my chunks: while chunk k is being finished, the tensor-memory loads
                // of chunk k + 1 are in flight.  `tcgen05.wait::ld` waits for every outstanding load, so it
                // comes right before the next chunk's loads are issued.
                uint32_t va[CW], ha[CW], vb[CW], hb[CW];
                auto issue = [&](int c, uint32_t (&v)[CW], uint32_t (&h)[CW]) {
                    tmem_load_chunk_nowait<CW>(tmem_acc + lane_bits + (uint32_t)(c * CW), v);
                    if (add_held) tmem_load_chunk_nowait<CW>(tmem_held + lane_bits + (uint32_t)(c * CW), h);
                };
                auto finish = [&](int c, uint32_t (&v)[CW], uint32_t (&h)[CW]) {
                    const uint32_t mask = valid ? realmask[c] : 0u;   // columns that are real pixels; the rest is zero padding
                    // (`h` is zero in a layer that adds nothing.  Padding columns are computed like the others but never
                    // stored: their rows of the operand buffer stay zero from the start, and what the held columns
                    // carry there only ever flows back into padding columns.)
#pragma unroll
                    for (int j = 0; j < CW; j++) {
                        float x = __uint_as_float(v[j]) + bias + __uint_as_float(h[j]);
                        if (relu) x = fmaxf(x, 0.f);
                        v[j] = __float_as_uint(x);
                    }
                    if (!last && has_block) {
                        // Four positions per store instruction: `stmatrix` writes four 8 x 16-byte matrices, and a
                        // 16-byte matrix row is exactly what four neighbouring lanes (channels) hold of one position,
                        // one 16-byte chunk of its 128-byte operand row.  Lane 8 k + r supplies the address of row r
                        // (channels 4 r .. 4 r + 3) of matrix k (position 4 m + k of the chunk), swizzled like the rest.
                        // One 32-bit store per position took four times the instructions and was the larger half of
                        // the epilogue's time.
                        uint32_t rounded[CW];
#pragma unroll
                        for (int j = 0; j < CW; j++) {
                            uint32_t u = v[j];
                            if ((u & 0x7F800000u) != 0x7F800000u) u += 0x1000u;
                            rounded[j] = u;
                        }
                        const uint32_t all = realmask[c];
#pragma unroll
                        for (int m = 0; m < CW / 4; m++) {
                            const uint32_t col = (uint32_t)(4 * m) + ((uint32_t)lane >> 3);
                            uint32_t addr = block_rows + ((uint32_t)c * CW + col) * 128u + ((((uint32_t)lane & 7u) ^ (col & 7u)) << 4);
                            if (!((all >> col) & 1u)) addr = dummy_rows + (((uint32_t)lane & 7u) << 4);
                            asm volatile("stmatrix.sync.aligned.m8n8.x4.shared.b16 [%0], {%1, %2, %3, %4};"
                                         ::"r"(addr), "r"(rounded[4 * m]), "r"(rounded[4 * m + 1]), "r"(rounded[4 * m + 2]), "r"(rounded[4 * m + 3])
                                         : "memory");
                        }
                    }
                    if (hold) tmem_store_chunk<CW>(tmem_held + lane_bits + (uint32_t)(c * CW), v);
                    if (to_global) {
#pragma unroll
                        for (int j = 0; j < CW; j++) {
                            if ((mask >> j) & 1u) {
                                const uint32_t info = colinfo[c * CW + j];
                                o_ptr[(img0 + ((info >> 16) & 0xFF)) * o_s0 + (int64_t)((info >> 8) & 0xFF) * o_s2 +
                                      (int64_t)(info & 0xFF) * o_s3] = __uint_as_float(v[j]);
                            }
                        }
                    }
                };
                // (not unrolled over the chunks: eight copies of the body made the epilogue's code so large that
                // the kernel's speed depended on where unrelated code happened to be placed, measured)
                if (!add_held) {
#pragma unroll
                    for (int j = 0; j < CW; j++) ha[j] = hb[j] = 0u;
                }
                if (half < chunks) issue(half, va, ha);
#pragma unroll 1
                for (int c = half; c < chunks; c += 2 * E) {
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (c + E < chunks) issue(c + E, vb, hb);
                    finish(c, va, ha);
                    if (c + E >= chunks) break;
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (c + 2 * E < chunks) issue(c + 2 * E, va, ha);
                    finish(c + E, vb, hb);
                }
                if (hold) asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            }
            if (trace) p.trace[l * 8 + 6] = clock64();
            if (!last) {
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(act_bar);
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"((uint32_t)p.tmem_cols) : "memory");
    }
}

}  // namespace

// ---------------------------------------------------------------- host side
static int round_up_int(int x, int to) { return (x + to - 1) / to * to; }

bool tc_chain_geometry(int h, int w, int64_t n_img, int c_blocks, ChainGeometry* out) {
    if (h < 1 || w < 1 || h > 254 || w > 254 || n_img < 1 || c_blocks < 1 || c_blocks > 4) return false;
    ChainGeometry best{};
    double best_cost = 1e300;
    // gx images side by side, gy such rows of images below one another
    for (int gx = 1; gx <= 16; gx++) {
        for (int gy = 1; gy <= 16; gy++) {
            ChainGeometry g{};
            g.gx = gx;
            g.gy = gy;
            g.per_cta = gx * gy;
            g.wp = gx * (w + 1);
            g.q_first = g.wp + 1;
            g.r_first = round_up_int(g.q_first, 8);
            const int q_last = ((gy - 1) * (h + 1) + h) * g.wp + (gx - 1) * (w + 1) + w;
            g.n_mma = round_up_int(q_last - g.q_first + 1, 16);
            if (g.n_mma > 256) break;
            g.rows_alloc = round_up_int(g.r_first + g.n_mma + g.wp + 2, 8);
            const int act_bytes = c_blocks * g.rows_alloc * 128;
            const int fixed = 1024 /* alignment */ + 16 * 8 + 32 + 1024 /* column table */ + 128 /* chunk masks */ + 24 /* poller's verdict */ + 128 /* dummy rows */;
            // the ring holds whole taps (c_blocks tiles each): two of them at least, four at most
            g.group = c_blocks;
            const int requests = std::min(4, (227 * 1024 - fixed - act_bytes) / (kTileBytes * g.group));
            if (requests < 2) break;
            g.slots = requests * g.group;
            g.smem_bytes = fixed + act_bytes + g.slots * kTileBytes;
            // per layer: 36 tiles x 4 MMAs (an MMA costs ~70 cycles up to N = 128, then grows with N), plus
            // the epilogue over the columns; CTAs run in waves of one per SM
            const double mma = std::max(70.0, 0.47 * g.n_mma + 16.0);
            const double per_layer = 144.0 * mma + 22.0 * g.n_mma + 900.0;
            const int64_t ctas = (n_img + g.per_cta - 1) / g.per_cta;
            const double cost = (double)((ctas + 147) / 148) * per_layer;
            if (cost < best_cost) {
                best_cost = cost;
                best = g;
            }
        }
    }
    if (best.per_cta == 0) return false;
    if (out) *out = best;
    return true;
}

struct ChainLaunch {
    CUtensorMap map_tiles;
    ChainKernelParams p;
    dim3 grid;
    int smem_bytes;
    int epilogue_warps;   // per lane quarter: the kernel variant
};

std::shared_ptr<void> chain_prepare(const ConvChainParams& c, uint32_t* status_word) {
    auto l = std::make_shared<ChainLaunch>();
    ChainKernelParams& p = l->p;
    memset(&p, 0, sizeof(p));
    int c_blocks_max = 1;
    p.total_tiles = 0;
    for (int i = 0; i < c.n_layers; i++) {
        c_blocks_max = std::max<int>(c_blocks_max, c.c_blocks[i]);
        p.total_tiles += ((c.flags[i] & kChainFlagPointwise) ? 1 : 9) * c.c_blocks[i];
        p.flags[i] = c.flags[i];
        p.c_blocks[i] = c.c_blocks[i];
    }
    c_blocks_max = std::max(c_blocks_max, (c.k + 31) / 32);
    ChainGeometry g;
    KN_CHECK(tc_chain_geometry(c.h, c.w, c.n, c_blocks_max, &g), KN_ERR_INTERNAL, "convolution chain does not fit");
    p.in = c.in;
    p.out = c.out;
    p.bias = c.bias;
    p.tiles = c.tiles;
    for (int i = 0; i < 4; i++) {
        p.s_in[i] = c.s_in[i];
        p.s_out[i] = c.s_out[i];
    }
    p.n_img = c.n;
    p.c_in = c.c_in;
    p.k = c.k;
    p.h = c.h;
    p.w = c.w;
    p.n_layers = c.n_layers;
    p.per_cta = g.per_cta;
    p.gx = g.gx;
    p.gy = g.gy;
    p.wp = g.wp;
    p.q_first = g.q_first;
    p.r_first = g.r_first;
    p.n_mma = g.n_mma;
    p.rows_alloc = g.rows_alloc;
    p.slots = g.slots;
    p.c_blocks_max = c_blocks_max;
    int cols = 2 * g.n_mma, tmem = 32;
    while (tmem < cols) tmem <<= 1;
    p.tmem_cols = tmem;
    p.status = status_word;
    KN_CHECK(c.n_heads >= 0 && c.n_heads <= kMaxChainHeads, KN_ERR_INTERNAL, "convolution chain with too many heads");
    p.n_heads = c.n_heads;
    for (int i = 0; i < c.n_heads; i++) {
        p.head_begin[i] = c.head_begin[i];
        p.head_out[i] = c.head_out[i];
        p.head_relu[i] = c.head_relu[i];
        for (int d = 0; d < 4; d++) p.head_s_out[i][d] = c.head_s_out[i][d];
    }
    p.head_begin[c.n_heads] = c.head_begin[c.n_heads];
    // one request per filter tap (all channel blocks of the tap, up to 64 KB): large requests stream at
    // about twice the rate of single 16 KB tiles
    p.group = g.group;
    p.slots = g.slots / p.group;
    // KN_CHAIN_TRACE=1 in the environment: the traced variant of the kernel stamps clock64 per layer in its first CTA
    // (MMA issuer: wait for the layer's input, all MMAs issued; first epilogue warp: accumulator ready, chunks
    // finished) and the table is printed when the process exits.  A measuring aid: the stamps cost a few percent.
    if (getenv("KN_CHAIN_TRACE") && p.n_layers <= kMaxChainLayers) {
        static long long* table = nullptr;
        static int layers = 0;
        if (!table && cudaHostAlloc((void**)&table, (size_t)kMaxChainLayers * 64, cudaHostAllocMapped) == cudaSuccess) {
            atexit([] {
                const long long* d = table;
                fprintf(stderr, "conv_chain_kernel, CTA 0, SM clock cycles per layer\n"
                                "layer  wait_input  issue_mmas  (of which filter waits)  accumulator_wait  epilogue_chunks  layer_period\n");
                for (int i = 0; i < layers; i++)
                    fprintf(stderr, "%5d  %10lld  %10lld  %23lld  %16lld  %15lld  %12lld\n", i, d[i * 8 + 1] - d[i * 8 + 0],
                            d[i * 8 + 2] - d[i * 8 + 1], d[i * 8 + 3], d[i * 8 + 5] - d[i * 8 + 4], d[i * 8 + 6] - d[i * 8 + 5],
                            i ? d[i * 8 + 1] - d[(i - 1) * 8 + 1] : 0);
            });
        }
        if (table) {
            memset(table, 0, (size_t)kMaxChainLayers * 64);
            layers = p.n_layers;
            p.trace = table;
        }
    }
    int64_t dims[3] = {32, 128, p.total_tiles}, strides[3] = {1, 32, 128 * 32};
    int box[3] = {32, 128, 1};
    l->map_tiles = tc_make_map(c.tiles, 3, dims, strides, box, true);
    l->grid = dim3((unsigned)((c.n + g.per_cta - 1) / g.per_cta), 1, 1);
    l->smem_bytes = g.smem_bytes;
    // Epilogue variants: the accumulator's columns are shared out in chunks among E warps per lane quarter.  Three
    // warps taking 16-column chunks when the chunk count divides by three (two 8x8 boards: 9 chunks, three each
    // instead of five and four), else two.  Four or six warps taking 8-column chunks exist as variants and measured
    // slower (two boards: 315 / 327 us against 314.5): the epilogue is bound by instruction issue, not by latency.
    // KN_CHAIN_EPILOGUE=<E> in the environment picks one (measuring).
    l->epilogue_warps = ((g.n_mma / 16) % 3 == 0) ? 3 : 2;
    if (const char* e = getenv("KN_CHAIN_EPILOGUE")) {
        const int v = atoi(e);
        if (v == 2 || v == 3 || v == 4 || v == 6) l->epilogue_warps = v;
    }
    return l;
}

int chain_launch(const void* launch, cudaStream_t stream) {
    const ChainLaunch& l = *(const ChainLaunch*)launch;
    static std::mutex mu;
    static bool done[64] = {false};
    int device = 0;
    cudaGetDevice(&device);
    {
        std::lock_guard<std::mutex> lock(mu);
        if (device >= 0 && device < 64 && !done[device]) {
            const void* variants[] = {
                (const void*)conv_chain_kernel<2, 16, false>, (const void*)conv_chain_kernel<3, 16, false>,
                (const void*)conv_chain_kernel<4, 8, false>,  (const void*)conv_chain_kernel<6, 8, false>,
                (const void*)conv_chain_kernel<2, 16, true>,  (const void*)conv_chain_kernel<3, 16, true>,
                (const void*)conv_chain_kernel<4, 8, true>,   (const void*)conv_chain_kernel<6, 8, true>,
            };
            for (const void* v : variants) {
                cudaError_t e = cudaFuncSetAttribute(v, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
                if (e != cudaSuccess) return (int)e;
            }
            done[device] = true;
        }
    }
    if (l.grid.x == 0) return 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = l.grid;
    cfg.blockDim = dim3(64 + 128 * l.epilogue_warps);
    cfg.dynamicSmemBytes = (size_t)l.smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    void* args[] = {(void*)&l.map_tiles, (void*)&l.p};
    const void* kernel = nullptr;
    const bool t = l.p.trace != nullptr;
    switch (l.epilogue_warps) {
        case 6: kernel = t ? (const void*)conv_chain_kernel<6, 8, true> : (const void*)conv_chain_kernel<6, 8, false>; break;
        case 4: kernel = t ? (const void*)conv_chain_kernel<4, 8, true> : (const void*)conv_chain_kernel<4, 8, false>; break;
        case 3: kernel = t ? (const void*)conv_chain_kernel<3, 16, true> : (const void*)conv_chain_kernel<3, 16, false>; break;
        default: kernel = t ? (const void*)conv_chain_kernel<2, 16, true> : (const void*)conv_chain_kernel<2, 16, false>; break;
    }
    return (int)cudaLaunchKernelExC(&cfg, kernel, args);
}

}  // namespace kn
