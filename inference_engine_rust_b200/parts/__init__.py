"""The parts layers are assembled from.  Importing this package registers the built-in
kinds: norm "rmsnorm", position "rope", mixer "attention", ffn "swiglu", block "prenorm",
head "linear"; norm "layernorm", block "hyper" (a residual of several streams), input "embed_norm",
head "softcap", ffn "moe", mixers "mlstm", "gated_delta" and "latent_attention"; block "outnorm" (the norm on a
sublayer's output), head "scaled", mixers "tied_kv_attention" (keys double as values), "rglru" (a gated linear
recurrence with a short convolution) and "parallel" (two mixers side by side); block "shared_norm" (one norm read by
both sublayers), mixer "gated_attention" (biases, a norm per head of q and k, a value size of its own, a sigmoid gate on
the heads), ffn "grouped_moe" (scores over all outputs or a sigmoid each, choice inside the best groups, experts that return
their input); mixer "wkv" (a matrix state with a decay per key channel, token shift); "tied_kv_attention" also takes a mask of
chunks, "latent_attention" also a rotated key part shared by the heads and a gate per head."""
from .base import (Block, FeedForward, Head, Mixer, Norm, Part, PositionEncoding, Runtime, StepContext, StepInput,
                   Workspace, part_class, register_part, unregister_part)
from .linear import Linear
from . import (norm, rope, attention, swiglu, block, head, inputs, moe, recurrent,  # noqa: F401  (registration)
               latent_attention, tied_attention, rglru, parallel, gated_attention)

__all__ = ["Block", "FeedForward", "Head", "Mixer", "Norm", "Part", "PositionEncoding", "Runtime",
           "StepContext", "StepInput", "Workspace", "part_class", "register_part", "unregister_part", "Linear"]
