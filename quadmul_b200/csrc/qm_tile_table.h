// Shape -> kernel plan for B200.  Replaces the reference's A40-tuned constexpr table
// (configs.cu:19-689) and its exact-match dispatch chain (kernel.cu:343-384): instead of 42
// hard-wired (M, N, K) triples and a silent no-op for anything else, every shape resolves to a
// plan, chosen by the rules below.
#pragma once
#include "qm_internal.h"
#include "tile_table.inc"  // generated: swept shapes and the cost-model coefficients of the decode kernel families

namespace qm {

struct PlanRule {
    int m_max;    // rule applies to m <= m_max (rows of C)
    int swap_ab;  // 1: B rows on the 128-wide UMMA-M axis, tokens on UMMA-N (decode form)
    int tile_n;   // UMMA N extent
    int cta_pair; // 1 or 2
};

// Ordered by m_max.  Decode-sized m (<= 64) puts the weights on the M axis so that a 128-row MMA is fully
// used by weight rows and only `tile_n` (>= m) columns are spent on tokens; it runs gemm_dec_kernel, which
// feeds the converted weights to the MMA from TMEM (measured against the all-shared-memory form of
// gemm_tc_kernel: 16 x 11008 x 4096 11.6 vs 12.5 us, 64 x 4096 x 4096 13.0 vs 14.8 us, 64 x 11008 x 4096
// 13.7 vs 15.5 us, equal at 16 x 4096 x 4096).  Everything larger runs
// the 256 x 256 CTA-pair tile: measured on B200 it beats the single-CTA 128 x 256 and both 128-wide
// forms at 8192^3 and at all four M = 2048 prefill shapes (python -m quadmul_b200.tune), because
// each SM converts and feeds only half of the B tile.
static const PlanRule kPlanRules[] = {
    {16, 1, 16, 1},
    {32, 1, 32, 1},
    {64, 1, 64, 1},
    {0x7FFFFFFF, 0, 256, 2},
};

// ---- decode shapes (m <= 64): which kernel family ----------------------------------------------------------------
// Three families take a product with few rows of A: gemm_rmma_kernel, gemv_kernel, gemm_dec_kernel.  A shape that was swept
// on B200 runs the family measured fastest there (exact-match entry of the generated table); any other shape runs the
// family whose modelled time -- a linear form in a few structural features, fitted to the same sweep -- is smallest.
// `quadmul_b200/tile_table_gen.py` holds the same feature expressions.
enum DecodeFamily : int { kFamNone = -1, kFamRmma = 0, kFamGemv = 1, kFamDec = 2 };

inline double decode_cost(int family, int m, int n, int k, int num_sms)
{
    const double mb = (double)n * k / 2 / 1e6;
    if (family == kFamRmma) {
        const double rounds = (double)(((n + 31) / 32 + num_sms - 1) / num_sms), tiles = (double)((m + 15) / 16), kq = k / 4096.0;
        const double half = m <= 8 ? 1.0 : 0.0;  // up to 8 rows of A: half as many MMAs per round
        const double *c = table::kRmmaCost;
        return c[0] + c[1] * rounds + c[2] * kq + c[3] * rounds * kq + c[4] * tiles + c[5] * rounds * tiles + c[6] * half +
               c[7] * rounds * kq * half;
    }
    if (family == kFamGemv) {
        const double *c = table::kGemvCost;
        return c[0] + c[1] * mb + c[2] * m * mb + c[3] * m;
    }
    const double *c = table::kDecCost[m <= 16 ? 0 : (m <= 32 ? 1 : 2)];
    return c[0] + c[1] * mb + c[2] * m + c[3] * m * mb;
}

// `ok[f]`: family f can take this call (shape limits and operand alignment).  Returns kFamNone when none can.
inline int choose_decode_family(int m, int n, int k, int num_sms, const bool (&ok)[3])
{
    if (num_sms == table::kSweepSms) {
        // swept shapes, sorted by (m, n, k): binary search
        int lo = 0, hi = table::kNumSwept - 1;
        while (lo <= hi) {
            const int mid = (lo + hi) / 2;
            const table::Swept &s = table::kSwept[mid];
            const int cmp = s.m != m ? (s.m < m ? -1 : 1) : (s.n != n ? (s.n < n ? -1 : 1) : (s.k != k ? (s.k < k ? -1 : 1) : 0));
            if (cmp == 0) {
                if (ok[s.family]) return s.family;
                break;
            }
            if (cmp < 0) lo = mid + 1;
            else hi = mid - 1;
        }
    }
    int best = kFamNone;
    double best_t = 0;
    for (int f = 0; f < 3; ++f) {
        if (!ok[f]) continue;
        const double t = decode_cost(f, m, n, k, num_sms);
        if (best == kFamNone || t < best_t) best = f, best_t = t;
    }
    return best;
}

inline bool tc_eligible(const GemmArgs &g)
{
    auto aligned16 = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    return g.k % 32 == 0 && g.k < 131072 && aligned16(g.A) && aligned16(g.B);
}

// Clusters of `size` CTAs (one CTA per SM) that run at once.  A cluster sits inside one GPC, so GPCs whose SM count is not
// a multiple of the size leave SMs unused: measured on B200 (148 SMs), 74 clusters of 2, 44 of 3, 32 of 4.  The dispatcher
// replaces this estimate by the driver's answer for the device at hand (dec_cluster_capacity).
inline int cluster_slots(int size, int num_sms)
{
    if (size <= 1) return num_sms;
    if (size == 2) return num_sms / 2;
    return size == 3 ? num_sms * 11 / 37 : num_sms * 8 / 37;
}

// The last round of whole 256 x 256 tiles over `units` CTA pairs holds tiles % units tiles.  When every one of them can be
// cut into at least two K partitions without exceeding the pairs (and a partition keeps at least two stages), that round runs
// as partitions instead: *tail_tiles tiles in *tail_split parts each.  Returns false when the tile list is left as it is.
inline bool tc2_tail_plan(int64_t tiles, int units, int stages, int *tail_tiles, int *tail_split)
{
    *tail_tiles = 0, *tail_split = 1;
    if (units < 1 || tiles <= units) return false;
    const int rest = (int)(tiles % units);
    int parts = rest > 0 ? units / rest : 0;
    if (parts > 8) parts = 8;
    if (parts > stages / 2) parts = stages / 2;
    if (parts < 2) return false;
    *tail_tiles = rest, *tail_split = parts;
    return true;
}

inline TcPlan plan_tc(int m, int n, int k, int num_sms)
{
    TcPlan p{256, 0, 1, 1, 0, 0, 1};
    for (const PlanRule &r : kPlanRules) {
        if (m <= r.m_max) {
            p.tile_n = r.tile_n;
            p.swap_ab = r.swap_ab;
            p.cta_pair = r.cta_pair;
            break;
        }
    }
    if (p.swap_ab) {
        // Decode form: few tiles, long K.  Split K so that the work items about fill the SMs; measured
        // best at 4 partitions for N = 4096 (32 tiles) and none for N = 11008 (86 tiles).
        const int tiles = ((n + 127) / 128) * ((m + p.tile_n - 1) / p.tile_n);
        const int num_kb = (k + 127) / 128;
        int s = tiles > 0 ? num_sms / tiles : 1;
        if (s > 4) s = 4;
        if (s > num_kb / 2) s = num_kb / 2;
        p.split_k = s < 1 ? 1 : s;
        p.a_tmem = 1;
        // Wide token tiles have large partial tiles (128 x 32 or 128 x 64 int32): their K partitions run as one
        // thread-block cluster and add up through its shared memory (32 x 4096 x 4096: 10.6 -> 9.1 us, 64 x 4096 x 4096:
        // 13.7 -> 11.4 us, 64 x 8192 x 8192: 18.5 -> 16.7 us).  With 16 tokens the scratch path is as fast (7.9 vs 8.1 us).
        if (p.tile_n >= 32 && p.split_k >= 2) p.stream_k = 2;
        if (p.stream_k == 2) {
            // One tile more than the device holds clusters and the launch takes two rounds (64 x 6144 x 4096, 48 tiles:
            // 23.5 us as clusters of 3, 12.6 us as clusters of 2): take the largest cluster that fits.
            while (p.split_k >= 2 && tiles > cluster_slots(p.split_k, num_sms)) --p.split_k;
            if (p.split_k < 2) p.stream_k = 0, p.split_k = 1;
        }
        if (p.tile_n == 16 && tiles > num_sms / 2) {
            // Enough tiles to put two smaller CTAs on every SM, which hide each other's pipeline bubbles:
            // 16 x 11008 x 4096 (86 tiles) 11.6 -> 10.3 us with 3 K partitions, 16 x 28672 x 8192 (224 tiles)
            // 29.6 -> 26.5 us.  Below that the CTAs of one launch end up paired on half of the SMs (16 x 4096 x 4096:
            // 9.0 us against 7.9 us with one CTA per SM).
            p.ctas_per_sm = 2;
            s = (2 * num_sms + tiles / 2) / tiles;
            if (s > 4) s = 4;
            if (s > num_kb / 2) s = num_kb / 2;
            p.split_k = s < 1 ? 1 : s;
        }
        // More tiles than CTA slots: whole tiles leave the last round partly empty, equal contiguous shares of the
        // (tile, K) work do not (16 x 57344 x 8192, 448 tiles: 48.2 us = 4.9 TB/s).
        if (tiles > num_sms * p.ctas_per_sm) p.stream_k = 1, p.split_k = 1;
    }
    if (!p.swap_ab) {
        // narrow outputs: do not spend a 256-wide tile on fewer columns
        if (n <= 16) p.tile_n = 16;
        else if (n <= 32) p.tile_n = 32;
        else if (n <= 64) p.tile_n = 64;
        else if (n <= 128) p.tile_n = 128;
        if (p.cta_pair == 2 && p.tile_n < 128) p.cta_pair = 1;
        // the 256 x 256 pair tile takes operand A through TMEM (gemm_tc2_kernel): 3.5 POPS against 2.3 POPS
        // for the all-shared-memory pair tile at 8192^3
        if (p.cta_pair == 2 && p.tile_n == 256) {
            p.a_tmem = 1;
            // Few tiles (short M and N): cut K so that more CTA pairs work; the partitions add into a zeroed C with
            // TMA reduce-add.  Measured: 128..256 x 4096 x 4096 (16 tiles) 17.1 -> 14.2 us with 4 partitions,
            // x 8192 x 8192 (32 tiles) 26.1 -> 21.2 us with 2; no gain once the tiles fill half of the pairs.
            const int tiles = ((m + 255) / 256) * ((n + 255) / 256);
            const int pairs = num_sms / 2, stages = (k + 255) / 256;
            if (tiles * 2 <= pairs) {
                int sk = pairs / tiles;
                if (sk > 4) sk = 4;
                if (sk > stages / 2) sk = stages / 2;
                p.split_k = sk < 1 ? 1 : sk;
            }
            // More tiles than pairs: a short last round is cut into K partitions (stream_k = 1 here means "split the
            // tail"; the launch decides with the number of pairs the device really runs at once).
            int tail_tiles, tail_split;
            if (p.split_k == 1 && tc2_tail_plan(tiles, pairs, stages, &tail_tiles, &tail_split)) p.stream_k = 1;
        }
    }
    return p;
}

}  // namespace qm
