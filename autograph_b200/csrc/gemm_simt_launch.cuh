// Host-side tile / split-k selection and launch of the SIMT tile engine.
#pragma once

#include "gemm_simt.cuh"

namespace ag {
namespace simt {

template <class Cfg, class AOp, class BOp, class Epi>
int launch_cfg(ag_device *dev, int M, int N, int K, int splits, int k_chunk, const AOp &A,
               const BOp &B, const Epi &E) {
    // m tiles on grid.x (up to 2^31 - 1), n tiles on grid.y.
    dim3 grid((unsigned)ceil_div(M, Cfg::BM), (unsigned)ceil_div(N, Cfg::BN), (unsigned)splits);
    AG_REQUIRE(grid.y <= 65535u && grid.z <= 65535u, AG_ERR_LIMIT,
               "problem too large for one launch (n tiles %u, splits %u)", grid.y, grid.z);
    gemm_simt_kernel<Cfg, AOp, BOp, Epi>
        <<<grid, Cfg::THREADS, 0, dev->stream>>>(M, N, K, k_chunk, A, B, E);
    AG_CHECK_LAUNCH();
    return AG_OK;
}

enum CfgId { kCfgL, kCfgM, kCfgXS, kCfgS16, kCfgS16s, kCfgS8 };

inline CfgId pick_cfg(int M, int N, int sms) {
    if (N <= 16 && ceil_div(M, 128) * 2 < sms) return kCfgS16s;
    if (N <= 8) return kCfgS8;
    if (N <= 16) return kCfgS16;
    int64_t tiles_l = ceil_div(M, CfgL::BM) * ceil_div(N, CfgL::BN);
    if (tiles_l >= sms) return kCfgL;
    int64_t tiles_m = ceil_div(M, 64) * ceil_div(N, 64);
    if (tiles_m * 2 >= sms) return kCfgM;
    return kCfgXS;
}

inline void cfg_dims(CfgId id, int &bm, int &bn) {
    switch (id) {
        case kCfgL: bm = CfgL::BM; bn = CfgL::BN; break;
        case kCfgM: bm = 64; bn = 64; break;
        case kCfgXS: bm = 32; bn = 32; break;
        case kCfgS16: bm = 128; bn = 16; break;
        case kCfgS16s: bm = 32; bn = 16; break;
        default: bm = 256; bn = 8; break;
    }
}

template <class AOp, class BOp, class Epi>
int launch_any(ag_device *dev, CfgId id, int M, int N, int K, int splits, int k_chunk,
               const AOp &A, const BOp &B, const Epi &E) {
    switch (id) {
        case kCfgL: return launch_cfg<CfgL>(dev, M, N, K, splits, k_chunk, A, B, E);
        case kCfgM: return launch_cfg<CfgM>(dev, M, N, K, splits, k_chunk, A, B, E);
        case kCfgXS: return launch_cfg<CfgXS>(dev, M, N, K, splits, k_chunk, A, B, E);
        case kCfgS16: return launch_cfg<CfgS16>(dev, M, N, K, splits, k_chunk, A, B, E);
        case kCfgS16s: return launch_cfg<CfgS16s>(dev, M, N, K, splits, k_chunk, A, B, E);
        default: return launch_cfg<CfgS8>(dev, M, N, K, splits, k_chunk, A, B, E);
    }
}

// Number of k splits for a problem that would otherwise leave most SMs idle.
// max_splits bounds the workspace (0 = never split).
inline int pick_splits(int64_t tiles, int K, int sms, int max_splits) {
    if (max_splits <= 1 || K < 256 || tiles * 2 > sms) return 1;
    int64_t want = ceil_div((int64_t)sms * 2, tiles);
    int64_t by_k = K / 64;  // at least 64 k per split
    int64_t s = want < by_k ? want : by_k;
    if (s > max_splits) s = max_splits;
    return s < 1 ? 1 : (int)s;
}

// C = A.B through epilogue E.  When the problem is split along k the partial
// sums go to the device workspace (or to `scratch` when the caller provides
// one of scratch_bytes) and a second kernel reduces them in a fixed order.
template <class AOp, class BOp, class Epi>
int gemm(ag_device *dev, int M, int N, int K, const AOp &A, const BOp &B, const Epi &E,
         bool allow_split, void *scratch = nullptr, size_t scratch_bytes = 0) {
    if (M <= 0 || N <= 0) return AG_OK;
    if (K >= 1 && K <= kSmallK && ceil_div(M, 32) * ceil_div(N, 32) <= dev->sm_count) {
        dim3 grid((unsigned)ceil_div(M, 32), (unsigned)ceil_div(N, 32));
        gemm_small_k_kernel<AOp, BOp, Epi><<<grid, 256, 0, dev->stream>>>(M, N, K, A, B, E);
        AG_CHECK_LAUNCH();
        return AG_OK;
    }
    CfgId id = pick_cfg(M, N, dev->sm_count);
    int bm, bn;
    cfg_dims(id, bm, bn);
    int64_t tiles = ceil_div(M, bm) * ceil_div(N, bn);
    int splits = allow_split ? pick_splits(tiles, K, dev->sm_count, 256) : 1;
    if (splits > 1 && scratch != nullptr) {
        int64_t fit = (int64_t)(scratch_bytes / (sizeof(float) * (size_t)M * (size_t)N));
        if (fit < splits) splits = (int)(fit < 1 ? 1 : fit);
    }
    if (splits <= 1) return launch_any(dev, id, M, N, K, 1, K > 0 ? K : 1, A, B, E);
    int k_chunk = (int)(ceil_div(ceil_div(K, splits), 32) * 32);  // multiple of every BK
    splits = (int)ceil_div(K, k_chunk);
    int64_t plane = (int64_t)M * N;
    void *ws = scratch;
    if (!ws) AG_TRY(workspace(dev, sizeof(float) * (size_t)plane * (size_t)splits, &ws));
    PartialEpilogue P{(float *)ws, plane, N};
    AG_TRY(launch_any(dev, id, M, N, K, splits, k_chunk, A, B, P));
    if (splits >= 16 && plane <= 32 * 4 * (int64_t)dev->sm_count) {
        splitk_reduce_small_kernel<Epi><<<(unsigned)ceil_div(plane, 32), 256, 0, dev->stream>>>(
            (const float *)ws, plane, splits, M, N, E);
    } else {
        int threads = 256;
        splitk_reduce_kernel<Epi><<<(unsigned)ceil_div(plane, threads), threads, 0, dev->stream>>>(
            (const float *)ws, plane, splits, M, N, E);
    }
    AG_CHECK_LAUNCH();
    return AG_OK;
}

}  // namespace simt
}  // namespace ag
