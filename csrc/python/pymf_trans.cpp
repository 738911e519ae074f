#include "pymf_parts.h"
void BindTrans(pybind11::module_ &) {}
