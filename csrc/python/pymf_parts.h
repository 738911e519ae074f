// Registration functions of the binding translation units.
#pragma once
#include <pybind11/pybind11.h>

#include "mf/mf.h"
#include "mf/mf_bm.h"

void BindBm(pybind11::module_ &m);      // pymf_bm.cpp
void BindShm(pybind11::module_ &m);     // pymf_shm.cpp
void BindTrans(pybind11::module_ &m);   // pymf_trans.cpp
void BindNative(pybind11::module_ &m);  // pymf_native.cpp
void BindOps(pybind11::module_ &m);     // pymf_ops.cpp
void BindTransport(pybind11::module_ &m);  // pymf_transport.cpp (adds to the "native" submodule, so it runs after BindNative)
