// Copy/cast kernels for source types int64..complex128.
#include "ew_cast.cuh"
namespace dpb {
void register_cast_b(EwTables &t) { reg_cast_rows<7>(t, std::make_integer_sequence<int, 7>()); }
}  // namespace dpb
