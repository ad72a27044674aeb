// Thin extern "C" doors onto the reference's own CPU codec.  TEST INFRASTRUCTURE ONLY.
//
// The build recipe (oracle/build_oracle.py) compiles this file four times, once per PART,
// with the reference checkout's packkv_cuda_ext/ and packkv_cuda_ext/include on the
// include path.  Each part textually includes ONE reference translation unit from where it
// lies in that checkout (nothing of the reference is copied into this repository) and
// instantiates its templates for the shapes the parity tests use.  The reference dispatches
// only (bits 4, block 64, hidden 1024/5120) for K and (bits 3, block 128, hidden 1024/5120)
// for V (k_encode_cpu.cpp:304-330, v_encode_cpu.cpp:319-345); the other combinations below
// are the same templates with other arguments.
//
// Output: oracle/_ref/libpackkv_ref.so, used to pin oracle/packkv_codec_oracle.c and to
// generate the committed fixtures.
#include <cstdint>
#include <cstddef>

#if PART == 1
#include "src/k_encode_cpu.cpp"
#define NS k_cpu
#define FN k_encode_cpu
#define ENCODE 1
#define HB 128
#elif PART == 2
#include "src/k_decode_cpu.cpp"
#define NS k_cpu
#define FN k_decode_cpu
#define ENCODE 0
#define HB 128
#elif PART == 3
#include "src/v_encode_cpu.cpp"
#define NS v_cpu
#define FN v_encode_cpu
#define ENCODE 1
#define HB 64
#elif PART == 4
#include "src/v_decode_cpu.cpp"
#define NS v_cpu
#define FN v_decode_cpu
#define ENCODE 0
#define HB 64
#elif PART == 5
#include "src/utils.cpp"
#endif

#if PART >= 1 && PART <= 4

#if ENCODE
#define CALL(BITS, HID, CB) \
    if (bits == BITS && hidden == HID && cb == CB) \
        return (long long)NS::FN<BITS, HID, HB, CB>(codes, stream, info, (size_t)ctx_len);
#else
#define CALL(BITS, HID, CB) \
    if (bits == BITS && hidden == HID && cb == CB) { \
        NS::FN<BITS, HID, HB, CB>(stream, info, codes, (size_t)ctx_len); return 0; }
#endif

#if HB == 128
#define FOR_CB(BITS, HID) CALL(BITS, HID, 32) CALL(BITS, HID, 64) CALL(BITS, HID, 128)
#else
#define FOR_CB(BITS, HID) CALL(BITS, HID, 128)
#endif
#define FOR_HID(BITS) FOR_CB(BITS, 128) FOR_CB(BITS, 256) FOR_CB(BITS, 1024)

extern "C" long long
#if PART == 1
ref_k_encode(const uint8_t *codes, uint8_t *stream, uint32_t *info,
#elif PART == 2
ref_k_decode(uint8_t *codes, const uint8_t *stream, const uint32_t *info,
#elif PART == 3
ref_v_encode(const uint8_t *codes, uint8_t *stream, uint32_t *info,
#else
ref_v_decode(uint8_t *codes, const uint8_t *stream, const uint32_t *info,
#endif
             long long ctx_len, long long hidden, int cb, int bits) {
    FOR_HID(2) FOR_HID(3) FOR_HID(4)
    return -1;  // combination not instantiated
}
#endif
