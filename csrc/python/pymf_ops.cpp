#include "pymf_parts.h"
void BindOps(pybind11::module_ &) {}
