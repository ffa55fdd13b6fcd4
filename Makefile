# Build of the sm_100a fluke library. Same targets and variables as the reference Makefile
# (:116-138): `make` (CPU only), `make cuda=1 CUDA_ARCH=...` -> lib/libfluke.a,
# `make shared cuda=1 CUDA_ARCH=...` -> lib/libfluke.so.
#
# CUDA_ARCH is accepted for compatibility with callers that pass the detected device arch
# (fluke_lib passes compute_100/sm_100), but the CUDA translation unit is ALWAYS compiled for
# sm_100a: tcgen05 and tensor memory only exist in the arch-specific target.
CC ?= gcc
AR ?= ar
CPPFLAGS += -I include/
CFLAGS += -g -Wall -O2 -fPIC -ffp-contract=off
DEPFLAGS = -MMD -MP
LDFLAGS += $(LIBS) -lm -lpthread
BUILD_DIR = lib

STATICLIB = $(BUILD_DIR)/libfluke.a
SHAREDLIB = $(BUILD_DIR)/libfluke.so

OBJ = $(BUILD_DIR)/misc.o $(BUILD_DIR)/error.o $(BUILD_DIR)/nn_cpu.o
GPU_OBJ =
SHARED_LINK = $(CC) -shared

ifdef asan
	CFLAGS += -fsanitize=address -fno-omit-frame-pointer
	LDFLAGS += -fsanitize=address -fno-omit-frame-pointer
endif

ifdef cuda
	CUDA_ROOT ?= /usr/local/cuda
	CUDA_LIB ?= $(CUDA_ROOT)/lib64
	CUDA_INC ?= $(CUDA_ROOT)/include
	NVCC ?= $(CUDA_ROOT)/bin/nvcc
	SM100_ARCH = -gencode arch=compute_100a,code=sm_100a
	CUDA_CFLAGS += -O3 -std=c++17 -lineinfo $(SM100_ARCH) -Xcompiler -Wall -Xcompiler -fPIC
	CUDA_LDFLAGS = -L$(CUDA_LIB) -lcudart_static -lrt -ldl
	CPPFLAGS += -DHAVE_CUDA=1 -I $(CUDA_INC)
	GPU_OBJ = $(BUILD_DIR)/fluke_sm100.o $(BUILD_DIR)/nn_gpu.o $(BUILD_DIR)/fused_i8.o \
	          $(BUILD_DIR)/fused_fp8.o $(BUILD_DIR)/lstm_host.o
	SHARED_LINK = $(NVCC) -shared $(SM100_ARCH)
	LDFLAGS += $(CUDA_LDFLAGS)
endif

ifdef debug
	CPPFLAGS += -DDEBUG=1
endif

SM100_SRC = fluke_b200/csrc/fluke_sm100_all.cu
SM100_DEPS = $(wildcard fluke_b200/csrc/*.cu fluke_b200/csrc/*.cuh fluke_b200/csrc/*.h)

PROBELIB = $(BUILD_DIR)/libfluke_probe.so
WAITPROBELIB = $(BUILD_DIR)/libfluke_waitprobe.so

.PHONY: all shared probe waitprobe clean distclean

all: $(STATICLIB)
shared: $(SHAREDLIB)
# tcgen05 issue-rate probe the benchmark compares the GEMM kernels with; not part of libfluke
probe: $(PROBELIB)

# test-only kernels that make the bounded device waits run out (tests/test_wait_timeout_gpu.py)
waitprobe: $(WAITPROBELIB)

$(WAITPROBELIB): tests/csrc/wait_probe.cu $(SM100_DEPS) | $(BUILD_DIR)
	$(NVCC) $(CUDA_CFLAGS) $(CPPFLAGS) -shared tests/csrc/wait_probe.cu -o $@ $(CUDA_LDFLAGS)

$(PROBELIB): fluke_b200/csrc/mma_peak_sm100.cu $(SM100_DEPS) | $(BUILD_DIR)
	$(NVCC) $(CUDA_CFLAGS) $(CPPFLAGS) -shared fluke_b200/csrc/mma_peak_sm100.cu -o $@ $(CUDA_LDFLAGS)

$(STATICLIB): $(OBJ) $(GPU_OBJ)
	rm -f $@
	$(AR) rcs $@ $(OBJ) $(GPU_OBJ)

$(SHAREDLIB): $(OBJ) $(GPU_OBJ)
	$(SHARED_LINK) -o $@ $(OBJ) $(GPU_OBJ) $(LDFLAGS)

$(BUILD_DIR)/%.o: src/%.c | $(BUILD_DIR)
	$(CC) $(CFLAGS) $(CPPFLAGS) $(DEPFLAGS) -c $< -o $@

$(BUILD_DIR)/fluke_sm100.o: $(SM100_SRC) $(SM100_DEPS) include/fluke/fluke.h | $(BUILD_DIR)
	$(NVCC) $(CUDA_CFLAGS) $(CPPFLAGS) -c $(SM100_SRC) -o $@

$(BUILD_DIR):
	mkdir -p $(BUILD_DIR)

-include $(BUILD_DIR)/*.d

clean:
	rm -rf $(BUILD_DIR)/*

distclean: clean
	git clean -f -X
