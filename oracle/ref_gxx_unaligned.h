/* TEST INFRASTRUCTURE ONLY -- force-included (g++ -include) into the reference's int8 depthwise
 * translation units by oracle/build_ref.sh, and into nothing else.
 *
 * The reference's depthwise kernel (src/kernel/elk_u8s8_depthwise_conv.hxx:171-214, 421-455) reads
 * 64 bytes starting at an arbitrary 16-byte pixel and at a weights table whose offset in the
 * workspace is 2*T*4 bytes past a 64-byte boundary (src/elx_int8_conv_direct_depthwise.cpp:178-181),
 * through _mm512_load_epi32 / _mm512_store_epi32.  The compiler the reference is normally built
 * with emits unaligned moves for those intrinsics; g++ emits aligned ones and the kernel faults.
 * Mapping the two intrinsics to their unaligned forms changes no arithmetic.
 */
#include <immintrin.h>
#define _mm512_load_epi32(p) _mm512_loadu_si512((const void *)(p))
#define _mm512_store_epi32(p, v) _mm512_storeu_si512((void *)(p), (v))
