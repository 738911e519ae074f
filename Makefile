# In-tree build of the native library and the Python extension.
#   make -j            → memfabric_hybrid_b200/lib/libmf_core.so + memfabric_hybrid_b200/_pymf*.so + csrc/test/mf_native_tests
#   make asan          → address+UB-sanitised host build of the native test binary
# CUDA sources are compiled for sm_100a only; host code links the static CUDA runtime so the library also loads on a
# machine without a GPU driver.
CUDA_HOME ?= /usr/local/cuda
NVCC      := $(CUDA_HOME)/bin/nvcc
PYTHON    ?= python
# The system compiler, deliberately not $CXX from the environment: a wrapper toolchain that links libstdc++ statically
# would put a second C++ runtime into a process that already has torch's, and the two do not mix.
CXX       := /usr/bin/g++

PY_INC    := $(shell $(PYTHON) -c "import sysconfig; print(sysconfig.get_paths()['include'])")
PYB_INC   := $(shell $(PYTHON) -c "import pybind11; print(pybind11.get_include())")
PY_EXT    := $(shell $(PYTHON) -c "import sysconfig; print(sysconfig.get_config_var('EXT_SUFFIX'))")
CUTLASS_INC ?= $(shell $(PYTHON) -c "import os, flashinfer; print(os.path.join(os.path.dirname(flashinfer.__file__), 'data', 'cutlass', 'include'))" 2>/dev/null)

BUILD     := build
OUTDIR    := memfabric_hybrid_b200/lib
CXXFLAGS  := -std=c++17 -O2 -g -fPIC -Wall -Wextra -Wno-unused-parameter -fvisibility=default -pthread \
             -fstack-protector-strong -D_FORTIFY_SOURCE=2 -I$(CUDA_HOME)/include -Iinclude -Icsrc
NVFLAGS   := -ccbin /usr/bin/g++ -std=c++17 -O3 -lineinfo -gencode arch=compute_100a,code=sm_100a -Xcompiler -fPIC -Iinclude -Icsrc \
             --expt-relaxed-constexpr -Xptxas -v
LDFLAGS   := -L$(CUDA_HOME)/lib64 -lcudart_static -ldl -lrt -pthread -Wl,-z,relro,-z,now

HOST_SRCS := $(wildcard csrc/util/*.cpp csrc/net/*.cpp csrc/transport/*.cpp csrc/store/*.cpp csrc/group/*.cpp csrc/hybm/*.cpp csrc/api/*.cpp)
CUDA_SRCS := $(wildcard csrc/kernels/*.cu)
HOST_OBJS := $(patsubst csrc/%.cpp,$(BUILD)/%.o,$(HOST_SRCS))
CUDA_OBJS := $(patsubst csrc/%.cu,$(BUILD)/%.cu.o,$(CUDA_SRCS))
TEST_SRCS := csrc/test/main.cpp

CORE      := $(OUTDIR)/libmf_core.so
PYMOD     := memfabric_hybrid_b200/_pymf$(PY_EXT)
TESTBIN   := csrc/test/mf_native_tests

all: $(CORE) $(PYMOD) $(TESTBIN)

$(BUILD)/%.o: csrc/%.cpp $(wildcard csrc/*/*.h include/mf/*.h)
	@mkdir -p $(dir $@)
	$(CXX) $(CXXFLAGS) -c $< -o $@

$(BUILD)/%.cu.o: csrc/%.cu $(wildcard csrc/*/*.h csrc/kernels/*.cuh include/mf/*.h include/mf/device/*.cuh)
	@mkdir -p $(dir $@)
	$(NVCC) $(NVFLAGS) -c $< -o $@ 2> $@.ptxas.log || (cat $@.ptxas.log; false)

$(CORE): $(HOST_OBJS) $(CUDA_OBJS)
	@mkdir -p $(OUTDIR)
	$(CXX) -shared -o $@.tmp $^ $(LDFLAGS) && mv -f $@.tmp $@

PY_SRCS   := $(wildcard csrc/python/*.cpp)
PY_OBJS   := $(patsubst csrc/%.cpp,$(BUILD)/%.py.o,$(PY_SRCS))
$(BUILD)/%.py.o: csrc/%.cpp $(wildcard csrc/*/*.h include/mf/*.h)
	@mkdir -p $(dir $@)
	$(CXX) $(CXXFLAGS) -fvisibility=hidden -I$(PY_INC) -I$(PYB_INC) -c $< -o $@

$(PYMOD): $(PY_OBJS) $(CORE)
	$(CXX) -shared -o $@.tmp $(PY_OBJS) -L$(OUTDIR) -lmf_core -Wl,-rpath,'$$ORIGIN/lib' $(LDFLAGS) && mv -f $@.tmp $@

$(TESTBIN): $(TEST_SRCS) $(CORE)
	$(CXX) $(CXXFLAGS) -o $@.tmp $(TEST_SRCS) -L$(OUTDIR) -lmf_core -Wl,-rpath,'$$ORIGIN/../../$(OUTDIR)' $(LDFLAGS) && mv -f $@.tmp $@

ASAN_FLAGS := -fsanitize=address,undefined -fno-omit-frame-pointer -O1
asan: $(CUDA_OBJS)
	@mkdir -p $(BUILD)/asan
	$(CXX) $(filter-out -O2 -D_FORTIFY_SOURCE=2,$(CXXFLAGS)) $(ASAN_FLAGS) -o $(BUILD)/asan/mf_native_tests_asan \
	    $(TEST_SRCS) $(HOST_SRCS) $(CUDA_OBJS) $(LDFLAGS)

# Mutation fuzzer of the parsers, built with the sanitizers (csrc/test/run_fuzz.sh runs it).
fuzz: $(CUDA_OBJS)
	@mkdir -p $(BUILD)/asan
	$(CXX) $(filter-out -O2 -D_FORTIFY_SOURCE=2,$(CXXFLAGS)) $(ASAN_FLAGS) -o $(BUILD)/asan/mf_fuzz \
	    csrc/test/fuzz_main.cpp $(HOST_SRCS) $(CUDA_OBJS) $(LDFLAGS)

# Libraries and tools are linked under a temporary name and renamed into place, so a reader of the tree (a packaging step, a
# process that has the old file mapped) never sees a half-written file.
# Example programs and tools that are built against the installed headers and library.
EXAMPLES := examples/bm_perf/bm_perf examples/bm_cpp/bm_example benchmarks/store_bench
examples: $(EXAMPLES)
examples/bm_perf/bm_perf: examples/bm_perf/bm_perf.cpp $(CORE)
	$(CXX) -std=c++17 -O2 -Iinclude -I$(CUDA_HOME)/include -o $@ $< -L$(OUTDIR) -lmf_core -Wl,-rpath,'$$ORIGIN/../../$(OUTDIR)' -L$(CUDA_HOME)/lib64 -lcudart -pthread
benchmarks/store_bench: benchmarks/store_bench.cpp $(CORE)
	$(CXX) -std=c++17 -O2 -Icsrc -Iinclude -o $@ $< -L$(OUTDIR) -lmf_core -Wl,-rpath,'$$ORIGIN/../$(OUTDIR)' -pthread
examples/bm_cpp/bm_example: examples/bm_cpp/main.cpp $(CORE)
	$(CXX) -std=c++17 -O2 -Iinclude -o $@ $< -L$(OUTDIR) -lmf_core -Wl,-rpath,'$$ORIGIN/../../$(OUTDIR)' -pthread

clean:
	rm -rf $(BUILD) $(CORE) $(PYMOD) $(TESTBIN)

.PHONY: all clean asan fuzz examples
