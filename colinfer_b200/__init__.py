"""colinfer_b200 -- the logits -> token path of the colinfer engine, rebuilt for B200 (sm_100a).

The package mirrors the reference's module layout for this path so that it is a drop-in:

    colinfer_b200.runtime.sampler   SamplerParams, apply_mask, sample        (engine/runtime/sampler.py)
    colinfer_b200.spec.accept       processed_probs, inverse_cdf, draw       (engine/spec/accept.py)
    colinfer_b200.spec.verify       spec_accept, spec_verify                 (accept block of engine/spec/mtp.py)
    colinfer_b200.kernels           ops().philox_uniform                     (engine/kernels, csrc/sampling.cu)

Everything runs in hand-written CUDA kernels behind a C ABI (include/colinfer_b200.h); there is no CPU path.
"""
__version__ = "1.0"
