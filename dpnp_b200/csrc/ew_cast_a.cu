// Copy/cast kernels for source types bool..uint32.
#include "ew_cast.cuh"
namespace dpb {
void register_cast_a(EwTables &t) { reg_cast_rows<0>(t, std::make_integer_sequence<int, 7>()); }
}  // namespace dpb
