// placeholder until the tcgen05 kernel lands: token chunks through the streaming kernel
#include "common.cuh"
namespace ob {
int64_t prefill_workspace_bytes(int64_t, int64_t, int64_t) { return 0; }
int launch_prefill(const FwdArgs &a)
{
    for (int64_t m0 = 0; m0 < a.M; m0 += ORTHO_B200_DECODE_MAX_M) {
        FwdArgs b = a;
        b.M = (a.M - m0 < ORTHO_B200_DECODE_MAX_M) ? (a.M - m0) : ORTHO_B200_DECODE_MAX_M;
        b.x = a.x + m0 * a.K;
        b.y = a.y + m0 * a.N;
        int st = launch_decode(b);
        if (st != ORTHO_B200_OK) return st;
    }
    return ORTHO_B200_OK;
}
}  // namespace ob
