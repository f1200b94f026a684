// The fused reduce-scatter + accumulate + re-encode + all-gather kernel with
// its traffic carried by bulk asynchronous copies (the TMA unit's untiled
// form, cp.async.bulk; no multicast anywhere): every warp pulls whole tiles
// of every rank's shard -- payload and scales, local or peer memory -- into a
// ring in shared memory, each tile's arrival counted by an mbarrier, and
// pushes the re-encoded tile to every rank's arena with bulk stores from a
// staging slot.  One elected lane issues the copies; the requests are whole
// contiguous rows (512 B - 1 KB of payload, 64 - 128 B of scales) instead of
// 16 bytes per lane, and none of it occupies the load / store units' miss
// queues.  The CTAs are launched to own their SMs (kExclusiveSharedBytes).
//
// Same arithmetic and tiling as bfp8_reduce_reencode_kernel: a sub-tile is 512
// values, a lane owns 16 consecutive ones.  Every wait is bounded: a tile that
// does not arrive within kBulkWaitLimit polls raises *finite_status (the step
// then fails closed on the host) and the warp stops taking tiles; before it
// leaves, it drains its outstanding stores.
#pragma once

#include "reduce_kernels.cuh"

namespace ngb {

constexpr unsigned kBulkWaitLimit = 1u << 22;     // polls of try_wait (each blocks for a while in hardware)

__device__ __forceinline__ unsigned shared_address(const void* p) {
    return static_cast<unsigned>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbarrier_init(void* barrier, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(shared_address(barrier)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbarrier_expect(void* barrier, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(shared_address(barrier)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbarrier_try_wait(void* barrier, unsigned parity) {
    unsigned done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(shared_address(barrier)), "r"(parity) : "memory");
    return done != 0;
}
// false when the wait ran out
__device__ __forceinline__ bool mbarrier_wait_bounded(void* barrier, unsigned parity) {
    for (unsigned poll = 0; poll < kBulkWaitLimit; ++poll)
        if (mbarrier_try_wait(barrier, parity)) return true;
    return false;
}
__device__ __forceinline__ void bulk_load(void* shared_destination, const void* global_source, unsigned bytes,
                                          void* barrier) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(shared_address(shared_destination)), "l"(global_source), "r"(bytes),
                   "r"(shared_address(barrier)) : "memory");
}
__device__ __forceinline__ void bulk_store(void* global_destination, const void* shared_source, unsigned bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                 ::"l"(global_destination), "r"(shared_address(shared_source)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int kPending>
__device__ __forceinline__ void bulk_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(kPending) : "memory");
}
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_shared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

// Bytes of one warp's share: kStages input slots of kRanks tiles, two output
// staging slots, kStages barriers.
template <int kBlock, int kRanks, int kStages, int kTile>
constexpr size_t bulk_warp_bytes() {
    constexpr size_t tile = kTile + 4 * (kTile / kBlock);
    return kStages * kRanks * tile + 2 * tile + ((kStages * 8 + 15) / 16) * 16;
}

template <int kBlock, int kRanks, bool kSquares, int kStages, int kWarps, int kTile>
__global__ void __launch_bounds__(kWarps * 32)
bfp8_reduce_reencode_bulk_kernel(EncodedShards shards, long long first_value, long long end_value,
                                 float reduction_scale, double* squared_sum, int* finite_status) {
    static_assert(kTile % 512 == 0 && kRanks > 0 && kStages >= 2, "whole sub-tiles, at least two stages");
    constexpr int kSubTiles = kTile / 512;
    constexpr int kTileScales = kTile / kBlock;
    constexpr int kScalesPerSub = 512 / kBlock;
    constexpr size_t kTileBytes = kTile + 4 * kTileScales;        // payload, then scales
    constexpr int kLanesPerBlock = kBlock / 16;
    extern __shared__ __align__(128) unsigned char bulk_shared[];
    const int lane = threadIdx.x & 31;
    const int warp_in_cta = threadIdx.x >> 5;
    constexpr size_t kWarpBytes = kStages * kRanks * kTileBytes + 2 * kTileBytes + ((kStages * 8 + 15) / 16) * 16;
    unsigned char* mine = bulk_shared + static_cast<size_t>(warp_in_cta) * kWarpBytes;
    unsigned char* in_ring = mine;                                              // [stage][rank][payload | scales]
    unsigned char* out_slots = mine + static_cast<size_t>(kStages) * kRanks * kTileBytes;   // [2][payload | scales]
    unsigned long long* full = reinterpret_cast<unsigned long long*>(out_slots + 2 * kTileBytes);

    const long long warp = static_cast<long long>(blockIdx.x) * kWarps + warp_in_cta;
    const long long warps = static_cast<long long>(gridDim.x) * kWarps;
    const long long span = end_value - first_value;
    const long long whole = span / kTile;                       // tiles moved by bulk copies
    double squares = 0.0;
    int non_finite = 0;

    if (lane == 0) {
        for (int s = 0; s < kStages; ++s) mbarrier_init(full + s, 1);
        fence_barrier_init();
    }
    __syncwarp();

    auto issue = [&](long long tile, int stage) {
        if (lane == 0 && tile < whole) {
            const long long base = first_value + tile * kTile;
            mbarrier_expect(full + stage, static_cast<unsigned>(kRanks * kTileBytes));
            #pragma unroll
            for (int k = 0; k < kRanks; ++k) {
                unsigned char* slot = in_ring + (static_cast<size_t>(stage) * kRanks + k) * kTileBytes;
                bulk_load(slot, shards.payload[k] + base, kTile, full + stage);
                bulk_load(slot + kTile, shards.scales[k] + base / kBlock, 4 * kTileScales, full + stage);
            }
        }
    };

    #pragma unroll
    for (int s = 0; s < kStages - 1; ++s) issue(warp + s * warps, s);
    int stage = 0, out_slot = 0;
    unsigned sequence = 0;
    bool alive = true;
    for (long long tile = warp; tile < whole && alive; tile += warps, ++sequence) {
        // refill the slot consumed in the previous iteration (all lanes are past it)
        __syncwarp();
        fence_async_shared();
        issue(tile + (kStages - 1) * warps, (stage + kStages - 1) % kStages);
        alive = mbarrier_wait_bounded(full + stage, (sequence / kStages) & 1u);
        alive = __all_sync(0xffffffffu, alive);
        if (!alive) { non_finite = 1; break; }
        // the staging slot about to be overwritten: its stores (two tiles ago) must have read it
        if (lane == 0) bulk_wait_read<1>();
        __syncwarp();
        unsigned char* out = out_slots + static_cast<size_t>(out_slot) * kTileBytes;
        #pragma unroll
        for (int sub = 0; sub < kSubTiles; ++sub) {
            float acc[16];
            #pragma unroll
            for (int k = 0; k < kRanks; ++k) {
                const unsigned char* slot = in_ring + (static_cast<size_t>(stage) * kRanks + k) * kTileBytes;
                const uint4 words = reinterpret_cast<const uint4*>(slot + sub * 512)[lane];
                const float scale = reinterpret_cast<const float*>(slot + kTile)[sub * kScalesPerSub + lane / kLanesPerBlock];
                non_finite |= bad_scale(scale);
                if (k == 0) accumulate16<true>(words, scale, acc);
                else accumulate16<false>(words, scale, acc);
            }
            uint4 packed;
            float scale;
            reencode16<kBlock, kSquares>(acc, reduction_scale, squares, non_finite, packed, scale);
            reinterpret_cast<uint4*>(out + sub * 512)[lane] = packed;
            if ((lane & (kLanesPerBlock - 1)) == 0)
                reinterpret_cast<float*>(out + kTile)[sub * kScalesPerSub + lane / kLanesPerBlock] = scale;
        }
        // make the staged tile visible to the copy unit, then push it everywhere
        fence_async_shared();
        __syncwarp();
        if (lane == 0) {
            const long long base = first_value + tile * kTile;
            for (int d = 0; d < shards.outputs; ++d) {
                bulk_store(shards.out_payload[d] + base, out, kTile);
                bulk_store(shards.out_scales[d] + base / kBlock, out + kTile, 4 * kTileScales);
            }
            bulk_commit();
        }
        stage = (stage + 1) % kStages;
        out_slot ^= 1;
    }
    // the ragged end (less than one tile): 512-value pieces with plain accesses,
    // dealt round-robin over the warps
    {
        const long long tail_start = first_value + whole * kTile;
        const long long pieces = (end_value - tail_start + 511) / 512;
        for (long long piece = warp; piece < pieces; piece += warps) {
            const long long base = tail_start + piece * 512;
            if (base + 512 <= end_value) {
                const long long at = base + lane * 16;
                float acc[16];
                #pragma unroll
                for (int k = 0; k < kRanks; ++k) {
                    const uint4 words = __ldcs(reinterpret_cast<const uint4*>(shards.payload[k] + at));
                    const float scale = __ldcs(shards.scales[k] + at / kBlock);
                    non_finite |= bad_scale(scale);
                    if (k == 0) accumulate16<true>(words, scale, acc);
                    else accumulate16<false>(words, scale, acc);
                }
                reencode_and_store<kBlock, kSquares>(shards, base, lane, acc, reduction_scale, squares, non_finite);
            } else {
                reduce_tile_scalar<kBlock, kSquares>(shards, kRanks, base, end_value, lane, reduction_scale,
                                                     squares, non_finite);
            }
        }
    }
    // Leave nothing in flight: stores complete; loads that were issued but not
    // consumed (only after a wait ran out) get one more bounded wait.
    if (lane == 0) bulk_wait_all();
    if (!alive) {
        // tiles `sequence` .. `sequence + kStages - 1` of this warp may still be landing
        for (unsigned i = sequence; i < sequence + kStages; ++i)
            if (warp + static_cast<long long>(i) * warps < whole)
                mbarrier_wait_bounded(full + i % kStages, (i / kStages) & 1u);
    }
    __syncwarp();
    if (finite_status != nullptr) {
        if (__any_sync(0xffffffffu, non_finite) && lane == 0) atomicExch(finite_status, 1);
    }
    if (kSquares) cta_accumulate(squares, squared_sum);
}

}  // namespace ngb
