/* Test infrastructure: just enough of the Metal Shading Language, as plain C++,
 * to compile the reference's SCALAR kernels of the attention path (head
 * RMSNorm x2, interleaved RoPE, AdaLN norm, gated residual) from the reference's
 * own shader text on a CPU.  Only tests and the golden-vector generator use it;
 * nothing in the product does.
 *
 * What is mapped:
 *   address spaces      device / constant / threadgroup -> nothing / const / a
 *                       buffer shared by the emulated threadgroup
 *   attributes          [[buffer(n)]], [[thread_position_in_grid]] ... are valid
 *                       C++11 attribute syntax and are ignored by the compiler
 *   types               uint, ushort, uint2, uint3
 *   as_type<T>(x)       bit cast
 *   fma(a, b, c)        fmaf (a real fused multiply-add)
 *   rsqrt(x)            1.0f / sqrtf(x): Metal leaves rsqrt's last bits to the
 *                       implementation; this is the correctly rounded choice
 *   threadgroup_barrier a std::barrier over the emulated threadgroup's threads
 * Multiply-add expressions that Metal's compiler may or may not contract are
 * compiled without contraction (-ffp-contract=off), the conservative reading.
 */
#ifndef QW_MSL_SHIM_H
#define QW_MSL_SHIM_H

#include <barrier>
#include <cmath>
#include <cstdint>
#include <cstring>

typedef uint32_t uint;
typedef uint16_t ushort;
struct uint2 { uint x, y; };
struct uint3 { uint x, y, z; };

template <typename To, typename From>
static inline To as_type(From value) {
    static_assert(sizeof(To) == sizeof(From), "as_type needs equal sizes");
    To out;
    std::memcpy(&out, &value, sizeof(out));
    return out;
}

static inline float fma(float a, float b, float c) { return std::fmaf(a, b, c); }
static inline float rsqrt(float x) { return 1.0f / std::sqrt(x); }

namespace mem_flags { enum flags { mem_none, mem_device, mem_threadgroup }; }

/* One emulated threadgroup at a time: its barrier and its shared arrays. */
namespace msl_emulation {
extern thread_local std::barrier<> *group_barrier;
}
static inline void threadgroup_barrier(mem_flags::flags) {
    if (msl_emulation::group_barrier) msl_emulation::group_barrier->arrive_and_wait();
}

#define kernel
#define device
#define constant const
/* `threadgroup float x[256];` inside a kernel: one array per threadgroup.  The
 * driver runs one threadgroup at a time, so a function-local static is that. */
#define threadgroup static

#endif
