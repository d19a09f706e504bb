"""One prefill step and a few eager decode steps of a synthetic Radanex (or Zedotar, Kulisun or Subivik) model: the program to put under
`ncu --metrics gpu__time_duration.sum` for a launch list of the sequence-state step (small: < 1 GB on the device).

    python scripts/seq_step_once.py [width] [batch] [context] [decode steps] [radanex|zedotar|kulisun|subivik]
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from umbrella_b200 import seq_bench  # noqa: E402

width, batch, ctx, steps = (int(x) for x in (sys.argv[1:5] + ["1024", "1", "512", "3"][len(sys.argv[1:5]):]))
if len(sys.argv) > 5 and sys.argv[5] == "zedotar":
    from umbrella_b200.models.zedotar import Zedotar as Family, spec_from_config  # noqa: E402
    spec = spec_from_config(seq_bench.zedotar_config(width, 8))
elif len(sys.argv) > 5 and sys.argv[5] == "kulisun":
    from umbrella_b200.models.kulisun import Kulisun as Family, spec_from_config  # noqa: E402
    spec = spec_from_config(seq_bench.kulisun_config(width, 8))
elif len(sys.argv) > 5 and sys.argv[5] == "subivik":
    from umbrella_b200.models.subivik import Subivik as Family, spec_from_config  # noqa: E402
    spec = spec_from_config(seq_bench.subivik_config(width, 8))
else:
    from umbrella_b200.models.radanex import Radanex as Family, spec_from_config  # noqa: E402
    spec = spec_from_config(seq_bench.radanex_config(width, 8))
m = Family(spec, device="cuda:0", dtype=torch.bfloat16, slots=batch, graph_decode=False, max_tokens=ctx + steps + 8)
m.alloc()
m.load_synthetic(7)
g = torch.Generator().manual_seed(0)
toks = lambda n: torch.randint(0, spec.vocab, (n,), generator=g).tolist()
slots = [m.cache.alloc_slot() for _ in range(batch)]
m.forward([(s, toks(ctx), [ctx - 1]) for s in slots])
torch.cuda.synchronize()
for _ in range(steps):
    m.forward([(s, toks(1), [0]) for s in slots])
torch.cuda.synchronize()
print("ok")
