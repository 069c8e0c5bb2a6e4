from grouped_gemm import _missing

gmm = permute = unpermute = _missing
