"""Small driver for profiler captures of whole decode steps.

    python -m nates_recipe_rs_b200.profile_decode <8b|70b> <batch> [steps] [layers]

Builds the random-init stack (optionally cut to `layers` layers so that a capture stays
small), fills the KV cache with seeded values and runs `steps` eager decode steps at the
end of the context, one kernel launch after the other (no CUDA graph), so that a launch
list attributes the time of a step to its kernels.
"""
import sys

import torch

from . import decoder as dec, quant_ops as ops


def main(argv):
    name, batch = argv[0], int(argv[1])
    steps = int(argv[2]) if len(argv) > 2 else 3
    torch.cuda.set_device(0)
    make = dec.config_8b if name == "8b" else dec.config_70b
    cfg = make(max_batch=batch)
    if len(argv) > 3:
        cfg.n_layers = int(argv[3])
    d = dec.Decoder(cfg)
    d.fill_cache(3)
    d.tokens.fill_(11)
    pos0 = cfg.ctx_len - steps - 1
    for i in range(steps):
        d.step(batch, pos0 + i)
        d.tokens.copy_(d.next_tokens)
    torch.cuda.synchronize()
    ops.check_launch()
    print("done", name, batch, "launch-visible layers:", cfg.n_layers)


if __name__ == "__main__":
    main(sys.argv[1:])
