"""The CUDA libraries of the engine: (source file, -D flags) pairs.  A model compiles what it
needs at first use; `all_libraries()` is everything, for the build check."""

ATTENTION_HEAD_DIMS = (16, 32, 48, 64, 80, 96, 112, 128)


def all_libraries():
    jobs = [("plain_kernels.cu", ()), ("gemm_tcgen05.cu", ()), ("gemv_fused.cu", ())]
    jobs += [("attention_mma.cu", (f"-DHEAD_DIM={d}",)) for d in ATTENTION_HEAD_DIMS]
    jobs += [("attention_tcgen05.cu", (f"-DHEAD_DIM={d}",)) for d in (64, 128)]
    jobs += [("attention_decode.cu", (f"-DHEAD_DIM={d}",)) for d in (64, 128)]
    return jobs
