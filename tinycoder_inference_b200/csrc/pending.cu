// Entry points whose kernels are still being built report TC_EUNSUPPORTED.
#include "tc_common.cuh"
extern "C" {
int tc_attn_decode_kv(const float *, const void *, const void *, float *, float *, float *, float *, uint32_t,
                      uint32_t, uint32_t, uint32_t, uint32_t, const uint32_t *, uint64_t, uint32_t, uint32_t,
                      float, int, uint8_t *, tc_stream) {
    tc::setError("tc_attn_decode_kv: not built yet");
    return TC_EUNSUPPORTED;
}
int tc_attn_prefill_f16_scratch_bytes(uint32_t, uint32_t, uint32_t, uint32_t, size_t *b) {
    if (b) *b = 0;
    return TC_EUNSUPPORTED;
}
int tc_attn_prefill_f16(const float *, const float *, const float *, float *, void *, size_t, uint32_t, uint32_t,
                        uint32_t, uint32_t, float, tc_stream) {
    tc::setError("tc_attn_prefill_f16: not built yet");
    return TC_EUNSUPPORTED;
}
int tc_attn_prefill_kv(const float *, const void *, const void *, float *, uint32_t, uint32_t, uint32_t, uint32_t,
                       uint32_t, const uint32_t *, uint64_t, float, int, tc_stream) {
    tc::setError("tc_attn_prefill_kv: not built yet");
    return TC_EUNSUPPORTED;
}
int tc_attn_prefill_i8(const float *, const int8_t *, const int8_t *, const float *, const float *, float *,
                       uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, const uint32_t *, uint64_t, float,
                       tc_stream) {
    tc::setError("tc_attn_prefill_i8: not built yet");
    return TC_EUNSUPPORTED;
}
}
