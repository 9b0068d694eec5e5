// Compile-once launcher of the fused all-reduce: every address, stride and flag
// location is resolved when the plan is built, so a steady-state call is one
// binding crossing followed by two or three kernel launches.
#pragma once

#include <torch/extension.h>

namespace lbc {
void bind_fused_plan(pybind11::module_& m);
}
