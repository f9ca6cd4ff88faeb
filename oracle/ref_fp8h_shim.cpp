// C entry points around the reference project's own host header fp8.h (decode, LUT, encoder).
// The header is compiled from where it lies in the reference checkout (-I<reference>); nothing of
// it is copied. TEST INFRASTRUCTURE ONLY: used to check the oracle against the reference's C++.
#include "fp8.h"

static const Fp8Format& pick(int fmt) { return fmt == 1 ? FMT_E5M2 : FMT_E4M3FN; }

extern "C" float ref_fp8_decode(unsigned char c, int fmt) { return fp8_decode(c, pick(fmt)); }
extern "C" unsigned char ref_fp8_encode(float x, int fmt) { return fp8_encode(x, pick(fmt)); }
extern "C" void ref_fp8_build_lut(int fmt, unsigned short* out256) { fp8_build_lut(pick(fmt), out256); }
