// Test-infrastructure only (never linked into the library): prints what NVIDIA CUTLASS's own host-side
// converters answer for a list of fp32 bit patterns read from stdin.  The reference's kernels get their
// e2m1 and ue4m3 rounding from exactly these templates - cutlass::NumericConverter<..., round_to_nearest>
// (kernels/src/reorder.cu:98-104 of ARCQuant) - so the tables this program produces pin the CPU oracle to
// the dependency itself rather than to a reading of the format definitions.
//
// stdin:  lines "e2m1 <hex>", "ue4m3 <hex>" (fp32 bit pattern) or "dec <code>" (ue4m3 code)
// stdout: one line per input: the resulting code, or for "dec" the fp32 bit pattern of the value
#include <cstdint>
#include <cstdio>
#include <cstring>

#include "cutlass/numeric_conversion.h"
#include "cutlass/numeric_types.h"
#include "cutlass/version.h"

int main() {
  cutlass::NumericConverter<cutlass::float_e2m1_t, float, cutlass::FloatRoundStyle::round_to_nearest> to_e2m1;
  cutlass::NumericConverter<cutlass::float_ue4m3_t, float, cutlass::FloatRoundStyle::round_to_nearest> to_ue4m3;
  fprintf(stderr, "cutlass %d.%d.%d\n", CUTLASS_MAJOR, CUTLASS_MINOR, CUTLASS_PATCH);
  char kind[16];
  unsigned int v;
  while (scanf("%15s %x", kind, &v) == 2) {
    float f;
    memcpy(&f, &v, 4);
    if (!strcmp(kind, "e2m1")) {
      printf("%u\n", (unsigned)to_e2m1(f).raw());
    } else if (!strcmp(kind, "ue4m3")) {
      printf("%u\n", (unsigned)to_ue4m3(f).raw());
    } else {
      const float d = float(cutlass::float_ue4m3_t::bitcast((uint8_t)v));
      unsigned int bits;
      memcpy(&bits, &d, 4);
      printf("%u\n", bits);
    }
  }
  return 0;
}
