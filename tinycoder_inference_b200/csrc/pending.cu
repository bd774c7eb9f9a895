// Entry points whose kernels are still being built report TC_EUNSUPPORTED.
#include "tc_common.cuh"
extern "C" {
int tc_attn_prefill_f16_scratch_bytes(uint32_t, uint32_t, uint32_t, uint32_t, size_t *b) {
    if (b) *b = 0;
    return TC_EUNSUPPORTED;
}
int tc_attn_prefill_f16(const float *, const float *, const float *, float *, void *, size_t, uint32_t, uint32_t,
                        uint32_t, uint32_t, float, tc_stream) {
    tc::setError("tc_attn_prefill_f16: not built yet");
    return TC_EUNSUPPORTED;
}
}
