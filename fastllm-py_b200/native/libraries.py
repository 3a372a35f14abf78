"""The list of CUDA libraries the engine can ask for: (source name, defines)."""
from .ops import BASE_LIBRARIES, BF16_LIBRARIES

# what parts name (`native_libraries`): every one of them, for a build of everything
PART_LIBRARIES = ["rope_kv", "attention_simt", "delta_rule", "latent_attention", "gemm_mma", "moe", "diff_attention",
                  "retention", "gated_block", "sink_attention", "norm_mix", "rglru", "gla"]

DEFAULT_HEAD_DIMS = (128,)


def all_libraries(head_dims=DEFAULT_HEAD_DIMS, latent_sizes=((512, 64),), diff_sizes=((64, 128),),
                  sink_sizes=((128, 128),)) -> list:
    """Every source; the attention kernels for `head_dims`, the tensor-core latent attention for
    `latent_sizes` ((latent size, rotated key size) pairs), the tensor-core differential attention for
    `diff_sizes` ((map size, value size) pairs) and the tensor-core sink attention for `sink_sizes`
    ((key size, value size) pairs), which are compiled per size."""
    from .attention import libraries as attention_libraries
    from .ops import diff_tc_library, latent_tc_library, sink_tc_library

    libs = [(name, {}) for name in BASE_LIBRARIES + PART_LIBRARIES + BF16_LIBRARIES]
    for d in head_dims:
        libs += attention_libraries(d)
    libs += [latent_tc_library(rank, rot) for rank, rot in latent_sizes]
    libs += [diff_tc_library(dim, vdim) for dim, vdim in diff_sizes]
    libs += [sink_tc_library(dim, vdim) for dim, vdim in sink_sizes]
    return libs


def libraries_for(dtype: str, head_dims=(), named=()) -> list:
    """What a model of this activation dtype needs, so that a first call can compile it side by
    side instead of one file after another: the libraries every model uses, those its parts name
    (`named`) and the attention builds for `head_dims`."""
    from .attention import handles, libraries as attention_libraries
    import torch

    libs = [(name, {}) for name in list(BASE_LIBRARIES) + sorted(set(named))]
    if dtype == "bfloat16":
        libs += [(name, {}) for name in BF16_LIBRARIES]
        for d in sorted(set(head_dims)):
            if handles(torch.bfloat16, d):
                libs += attention_libraries(d)
    return libs
