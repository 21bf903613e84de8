# Builds the library and its command-line tools for sm_100a.
#   make -j8            -> nccl_b200/lib/libnccl_b200.so + bin/ncclparam + bin/ncclras + plugins + bin/examples/*
#   make SAN=address    -> host code instrumented (CPU-only tests)
CUDA_HOME ?= /usr/local/cuda
NVCC      ?= $(CUDA_HOME)/bin/nvcc
CXX       ?= g++
BUILD     ?= build
LIBDIR    := nccl_b200/lib
BINDIR    := nccl_b200/bin

GENCODE   := -gencode arch=compute_100a,code=sm_100a
CXXFLAGS  := -std=c++17 -O2 -g -fPIC -Wall -Wno-unused-function -Wno-sign-compare \
             -Iinclude -Isrc -I$(CUDA_HOME)/include -pthread
NVCCFLAGS := -std=c++17 -O3 -lineinfo $(GENCODE) -Xcompiler -fPIC -Iinclude -Isrc \
             --expt-relaxed-constexpr -Xptxas -v $(EXTRA_NVCCFLAGS)
ifdef SAN
CXXFLAGS  += -fsanitize=$(SAN) -fno-omit-frame-pointer
LDSAN     := -fsanitize=$(SAN)
endif

HOST_SRCS := $(wildcard src/core/*.cc src/host/*.cc src/comm/*.cc src/mem/*.cc src/sched/*.cc \
               src/topo/*.cc src/transport/*.cc src/plugin/*.cc src/ras/*.cc src/ep/*.cc src/tp/*.cc \
               src/contrib/*.cc)
CU_SRCS   := $(wildcard src/kernels/*.cu src/ep/*.cu src/tp/*.cu src/contrib/*.cu)
HOST_OBJS := $(HOST_SRCS:%.cc=$(BUILD)/%.o)
CU_OBJS   := $(CU_SRCS:%.cu=$(BUILD)/%.cu.o)

LIB := $(LIBDIR)/libnccl_b200.so
TOOLS := $(patsubst tools/%.cc,$(BINDIR)/%,$(wildcard tools/*.cc))
PLUGIN_SRCS := $(wildcard plugins/*/*.cc)
PLUGINS := $(patsubst plugins/%.cc,$(LIBDIR)/plugins/%.so,$(PLUGIN_SRCS))

EXAMPLES := $(patsubst examples/%.cu,$(BINDIR)/examples/%,$(wildcard examples/*.cu))

IRLIB := $(LIBDIR)/libnccl_device_c.a

PERFLOOP := $(LIBDIR)/libperf_loop.so

all: $(LIB) $(TOOLS) plugins examples ir $(PERFLOOP)

# the loop of collective calls that the timing harness runs outside the interpreter (knows no library: entry points come in as addresses)
$(PERFLOOP): tools/perf_loop.c
	@mkdir -p $(LIBDIR)
	$(CC) -O2 -fPIC -shared -fvisibility=hidden $< -o $@

GIT_VERSION := $(shell git describe --always --dirty 2>/dev/null || echo unknown)
$(BUILD)/src/core/version.o: CXXFLAGS += -DB200_GIT_VERSION='"$(GIT_VERSION)"'

$(BUILD)/%.o: %.cc $(wildcard include/*.h src/*/*.h)
	@mkdir -p $(dir $@)
	$(CXX) $(CXXFLAGS) -c $< -o $@

$(BUILD)/%.cu.o: %.cu $(wildcard include/*.h include/nccl_device/*.h src/*/*.h src/*/*.cuh)
	@mkdir -p $(dir $@)
	$(NVCC) $(NVCCFLAGS) -c $< -o $@ 2> $@.ptxas.log || (cat $@.ptxas.log; exit 1)

$(LIB): $(HOST_OBJS) $(CU_OBJS)
	@mkdir -p $(LIBDIR)
	$(NVCC) -shared $(GENCODE) -o $@ $^ -cudart static -Xcompiler -pthread -Xlinker -Bsymbolic -ldl -lrt $(if $(SAN),-Xcompiler $(LDSAN))

$(BINDIR)/%: tools/%.cc $(LIB)
	@mkdir -p $(BINDIR)
	$(CXX) $(CXXFLAGS) $< -o $@ -L$(LIBDIR) -lnccl_b200 -Wl,-rpath,'$$ORIGIN/../lib' -ldl $(LDSAN)

examples: $(EXAMPLES)
$(BINDIR)/examples/%: examples/%.cu examples/common.h $(LIB) $(wildcard include/*.h include/nccl_device/*.h)
	@mkdir -p $(dir $@)
	$(NVCC) -std=c++17 -O2 -lineinfo $(GENCODE) -Iinclude $< -o $@ -L$(LIBDIR) -lnccl_b200 -Xlinker -rpath -Xlinker '$$ORIGIN/../../lib' -Xcompiler -pthread

# device API as C symbols carrying link-time-optimisation IR, for compilers of kernel languages (link with -dlto / nvJitLink)
ir: $(IRLIB)
$(IRLIB): bindings/ir/nccl_device_c.cu bindings/ir/nccl_device_c.h $(wildcard include/*.h include/nccl_device/*.h)
	@mkdir -p $(LIBDIR) $(BUILD)/bindings/ir
	$(NVCC) -std=c++17 -O3 -gencode arch=compute_100a,code=lto_100a -dc -Iinclude -Ibindings/ir $< -o $(BUILD)/bindings/ir/nccl_device_c.o
	rm -f $@ && ar rcs $@ $(BUILD)/bindings/ir/nccl_device_c.o

plugins: $(PLUGINS)
$(LIBDIR)/plugins/%.so: plugins/%.cc $(wildcard include/*.h include/plugin/*.h)
	@mkdir -p $(dir $@)
	$(CXX) $(CXXFLAGS) -shared $< -o $@

# make install PREFIX=/opt/nccl_b200 : library, headers, tools, plugins and a pkg-config file
PREFIX ?= /usr/local
install: all
	install -d $(DESTDIR)$(PREFIX)/lib/pkgconfig $(DESTDIR)$(PREFIX)/lib/nccl_b200/plugins $(DESTDIR)$(PREFIX)/bin \
	           $(DESTDIR)$(PREFIX)/include/nccl_device $(DESTDIR)$(PREFIX)/include/plugin
	install -m 755 $(LIB) $(DESTDIR)$(PREFIX)/lib/
	install -m 755 $(TOOLS) $(DESTDIR)$(PREFIX)/bin/
	install -m 644 include/*.h $(DESTDIR)$(PREFIX)/include/
	install -m 644 include/nccl_device/*.h $(DESTDIR)$(PREFIX)/include/nccl_device/
	install -m 644 include/plugin/*.h $(DESTDIR)$(PREFIX)/include/plugin/
	install -m 644 $(IRLIB) $(DESTDIR)$(PREFIX)/lib/
	install -m 644 bindings/ir/nccl_device_c.h $(DESTDIR)$(PREFIX)/include/
	cp -r $(LIBDIR)/plugins/. $(DESTDIR)$(PREFIX)/lib/nccl_b200/plugins/
	printf 'prefix=%s\nlibdir=$${prefix}/lib\nincludedir=$${prefix}/include\n\nName: nccl_b200\nDescription: collective communication library for B200 with the NCCL host API\nVersion: 2.30.7\nLibs: -L$${libdir} -lnccl_b200\nCflags: -I$${includedir}\n' '$(PREFIX)' > $(DESTDIR)$(PREFIX)/lib/pkgconfig/nccl_b200.pc

clean:
	rm -rf $(BUILD) $(LIBDIR) $(BINDIR)

.PHONY: all clean plugins examples install
