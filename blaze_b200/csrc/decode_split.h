// decode_split.h -- how the skinny-M kernels split K across CTAs; shared by the plan path and the
// allocation-free entry point so that both partition K identically (bit-identical results).
#pragma once

#include <cstdlib>

namespace blz {

// largest K split the skinny-M kernel supports for an instruction N of 16 / 32 / 64 (the partial
// sums of the other splits must fit the leader's stage buffers)
inline int decode_max_split(int mma_n) { return mma_n <= 16 ? 8 : mma_n <= 32 ? 4 : 2; }

// BLZ_DECODE_SPLIT=n forces the K split of every skinny-M launch (tuning); 0 / unset = the rule below.
inline int decode_split_override() {
    const char* v = getenv("BLZ_DECODE_SPLIT");
    return (v && *v) ? atoi(v) : 0;
}

// Smallest power-of-two split that gives at least 0.6 CTAs per SM (measured: 96 CTAs of 16 stages
// beat 192 of 8 on 148 SMs; 32 CTAs lose to 128), capped by `max_split`, by two
// pipeline stages per split and by "no split is empty".  `forced` > 0 overrides the first rule.
inline int decode_pick_split(int n_tiles, int k_stages_total, int num_sms, int max_split, int forced) {
    int s = 1;
    if (forced > 0) { while (s * 2 <= forced) s *= 2; }
    else { while (s < 8 && n_tiles * s * 10 < num_sms * 6) s *= 2; }
    while (s > max_split) s /= 2;
    while (s > 1 && k_stages_total / s < 2) s /= 2;
    while (s > 1 && (s - 1) * ((k_stages_total + s - 1) / s) >= k_stages_total) s /= 2;
    return s;
}

// W4A16 skinny-M kernel: consecutive weight tiles one CTA takes.  The kernel holds one CTA per SM, so a
// grid beyond one wave costs a second kernel time; without a K split the CTAs then share the tiles evenly,
// up to what the accumulator columns hold (two tiles for an instruction N of 16, one above).  `forced` > 0
// overrides the choice (still clamped to what the kernel supports).
inline int decode_tiles_per_cta(int n_tiles, int num_sms, int mma_n, int split, int forced) {
    const int t_max = mma_n <= 16 ? 2 : 1;
    int t = forced;
    if (t <= 0) t = (split == 1 && n_tiles > num_sms) ? (n_tiles + num_sms - 1) / num_sms : 1;
    return t > t_max ? t_max : t;
}

}  // namespace blz
