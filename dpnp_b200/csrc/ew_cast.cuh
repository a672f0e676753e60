// Copy/cast table population, split by source-type range so that two
// translation units share the compile time.
#pragma once
#include "ew_register.cuh"
namespace dpb {
template <int BYTES> constexpr int log2_bytes()
{
    return BYTES == 1 ? 0 : BYTES == 2 ? 1 : BYTES == 4 ? 2 : BYTES == 8 ? 3 : 4;
}
template <int TS, int TD> void reg_cast_one(EwTables &t)
{
    using S = type_of_t<TS>;
    using D = type_of_t<TD>;
    if constexpr (TS == TD) t.cast[TS][TD] = &ew_entry<CopyF<sizeof(S)>>;
    else t.cast[TS][TD] = &ew_entry<CastF<S, D>>;
}
template <int TS, int... TD> void reg_cast_row(EwTables &t, std::integer_sequence<int, TD...>)
{
    (reg_cast_one<TS, TD>(t), ...);
}
template <int FIRST, int... I> void reg_cast_rows(EwTables &t, std::integer_sequence<int, I...>)
{
    (reg_cast_row<FIRST + I>(t, std::make_integer_sequence<int, DPB_NUM_TYPES>()), ...);
}
}  // namespace dpb
