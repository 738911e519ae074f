#include "pymf_parts.h"
void BindShm(pybind11::module_ &) {}
