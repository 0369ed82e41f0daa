# Builds the sm_100a library, the per-stage command-line programs and the oracle.
#   make lib        ft_gemm_b200/lib/libft_gemm_b200.so   (C-ABI of include/ft_gemm.h)
#   make cli        build/stage_abft_fp8_gemm, build/fault_campaign, build/cublaslt_fp8_bench
#   make oracle     oracle/_build/libftq_oracle.so (CPU checker; test infrastructure)
#   make fault_campaign FAULT_TRIALS=1000   (mirrors the reference Makefile's campaign target)
NVCC      ?= nvcc
ARCH      ?= -gencode arch=compute_100a,code=sm_100a
NVCCFLAGS ?= -O3 -std=c++17 -lineinfo $(ARCH) -Xcompiler -fPIC -Xptxas -v
CSRC      := ft_gemm_b200/csrc
LIB       := ft_gemm_b200/lib/libft_gemm_b200.so
OBJS      := build/obj/prepare.o build/obj/prepare_mma.o build/obj/abft_gemm.o build/obj/api.o build/obj/noalloc.o build/obj/ft_attention.o build/obj/ft_attention_split.o build/obj/api_attention.o build/obj/gemm_softmax.o
HDRS      := include/ft_gemm.h include/ft_attention.h include/ft_gemm_softmax.h $(CSRC)/kernels.h $(CSRC)/attention_kernels.h $(CSRC)/attention_device.cuh $(CSRC)/abft_tile_check.cuh $(CSRC)/sm100_ptx.cuh

# the campaign the 100 % single-fault correction claim is quoted on: 8192^3, N(0,1) inputs, 1000 single faults U[1,256]
# with random sign + 50 double faults, relative tolerance 2e-6 (the reference's default 2e-5 puts the threshold near 6.7
# at K = 8192 with these inputs, above ~2 % of the injected magnitudes; FAULT_REL_TOL=0.00002 runs that configuration)
FAULT_SIZE      ?= 8192
FAULT_DIST      ?= normal
FAULT_TRIALS    ?= 1000
FAULT_DOUBLES   ?= 50
FAULT_MIN_VALUE ?= 1
FAULT_MAX_VALUE ?= 256
FAULT_SEED      ?= 12345
FAULT_REL_TOL   ?= 0.000002

all: lib cli oracle

lib: $(LIB)

build/obj/%.o: $(CSRC)/%.cu $(HDRS)
	@mkdir -p build/obj
	$(NVCC) $(NVCCFLAGS) -c -o $@ $<

$(LIB): $(OBJS)
	@mkdir -p ft_gemm_b200/lib
	$(NVCC) $(ARCH) -shared -o $@ $(OBJS)

cli: build/stage_abft_fp8_gemm build/fault_campaign build/cublaslt_fp8_bench build/ft_flash_attention build/gemm_softmax_abft

build/stage_abft_fp8_gemm: $(CSRC)/cli/stage_abft_fp8_gemm.cpp $(CSRC)/cli/cli_common.h $(HDRS) $(LIB)
	$(NVCC) -O2 -std=c++17 -Wno-deprecated-gpu-targets -Iinclude -o $@ $< -Lft_gemm_b200/lib -lft_gemm_b200 -lnccl -Xlinker -rpath -Xlinker '$$ORIGIN/../ft_gemm_b200/lib'

build/fault_campaign: $(CSRC)/cli/fault_campaign.cpp $(CSRC)/cli/cli_common.h $(HDRS) $(LIB)
	$(NVCC) -O2 -std=c++17 -Wno-deprecated-gpu-targets -Iinclude -o $@ $< -Lft_gemm_b200/lib -lft_gemm_b200 -Xlinker -rpath -Xlinker '$$ORIGIN/../ft_gemm_b200/lib'

build/ft_flash_attention: $(CSRC)/cli/ft_flash_attention.cpp $(CSRC)/cli/cli_common.h $(HDRS) $(LIB)
	$(NVCC) -O2 -std=c++17 -Wno-deprecated-gpu-targets -Iinclude -o $@ $< -Lft_gemm_b200/lib -lft_gemm_b200 -Xlinker -rpath -Xlinker '$$ORIGIN/../ft_gemm_b200/lib'

build/gemm_softmax_abft: $(CSRC)/cli/gemm_softmax_abft.cpp $(CSRC)/cli/cli_common.h $(HDRS) $(LIB)
	$(NVCC) -O2 -std=c++17 -Wno-deprecated-gpu-targets -Iinclude -o $@ $< -Lft_gemm_b200/lib -lft_gemm_b200 -Xlinker -rpath -Xlinker '$$ORIGIN/../ft_gemm_b200/lib'

build/cublaslt_fp8_bench: $(CSRC)/cli/cublaslt_fp8_bench.cpp $(CSRC)/cli/cli_common.h $(HDRS) $(LIB)
	$(NVCC) -O2 -std=c++17 -Wno-deprecated-gpu-targets -Iinclude -o $@ $< -Lft_gemm_b200/lib -lft_gemm_b200 -lcublasLt -lcublas -Xlinker -rpath -Xlinker '$$ORIGIN/../ft_gemm_b200/lib'

# Diagnostic build of the attention kernel with its timeline trace compiled in (FT_TRACE in ft_attention_split.cu); the
# product library is not touched:  make trace && ./build/trace/ft_flash_attention --batch 4 --heads 32 --sequence 4096 --trace
TRACE_OBJS := $(filter-out build/obj/ft_attention_split.o,$(OBJS)) build/trace/ft_attention_split.o
trace: build/trace/ft_flash_attention

build/trace/ft_attention_split.o: $(CSRC)/ft_attention_split.cu $(HDRS)
	@mkdir -p build/trace
	$(NVCC) $(NVCCFLAGS) -DFT_ATTENTION_TRACE -c -o $@ $<

build/trace/libft_gemm_b200.so: $(TRACE_OBJS)
	$(NVCC) $(ARCH) -shared -o $@ $(TRACE_OBJS)

build/trace/ft_flash_attention: $(CSRC)/cli/ft_flash_attention.cpp $(CSRC)/cli/cli_common.h $(HDRS) build/trace/libft_gemm_b200.so
	$(NVCC) -O2 -std=c++17 -Wno-deprecated-gpu-targets -DFT_ATTENTION_TRACE -Iinclude -o $@ $< -Lbuild/trace -lft_gemm_b200 -Xlinker -rpath -Xlinker '$$ORIGIN'

oracle:
	$(MAKE) -C oracle

fault_campaign: build/fault_campaign
	./build/fault_campaign --m $(FAULT_SIZE) --n $(FAULT_SIZE) --k $(FAULT_SIZE) --dist $(FAULT_DIST) --warmup 1 --repeat 1 \
	  --rel-tol $(FAULT_REL_TOL) --fault-min-value $(FAULT_MIN_VALUE) --fault-max-value $(FAULT_MAX_VALUE) \
	  --fault-trials $(FAULT_TRIALS) --double-trials $(FAULT_DOUBLES) --fault-seed $(FAULT_SEED)

clean:
	rm -rf build/obj

.PHONY: trace all lib cli oracle fault_campaign clean
