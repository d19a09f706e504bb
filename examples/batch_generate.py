"""Batched generation with a sequence-state decoder through the front-end surface: ``AutoEngine.from_config(device,
engine="batch", model=DIR)`` -> ``initialize()`` -> ``generate_batch(prompts)``.

    python examples/batch_generate.py --model DIR [--dtype bfloat16|float32] [--prompts 8] [--prompt-len 128]
                                      [--max-new-tokens 64] [--temperature 0.0]
    python examples/batch_generate.py --synthetic-width 1024          # no checkpoint: seeded random weights

``--model`` is a directory with config.json and model.safetensors; the model class is chosen by config.json's
``architecture``.  Prompts are random token ids (pass text through ``engine.generate(context=...)`` with a tokenizer).
"""
import argparse
import json
import os
import sys
import tempfile
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from umbrella_b200.speculation.auto_engine import AutoEngine  # noqa: E402

ap = argparse.ArgumentParser()
ap.add_argument("--config", default=None, help="an engine config such as configs/b200_batch_radanex.json, configs/b200_batch_zedotar.json, configs/b200_batch_kulisun.json or configs/b200_batch_subivik.json")
ap.add_argument("--model", default=None)
ap.add_argument("--synthetic-width", type=int, default=0, help="build a synthetic config of this width instead")
ap.add_argument("--family", default="radanex", choices=["radanex", "zedotar", "kulisun", "subivik"], help="family of the synthetic config")
ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
ap.add_argument("--prompts", type=int, default=8)
ap.add_argument("--prompt-len", type=int, default=128)
ap.add_argument("--max-new-tokens", type=int, default=64)
ap.add_argument("--temperature", type=float, default=0.0)
args = ap.parse_args()

config = {"engine": "batch", "dtype": args.dtype, "max_batch": args.prompts, "temperature": args.temperature}
if args.config:
    config.update(json.load(open(args.config)))
if args.model:
    config["model"] = args.model
if args.synthetic_width:
    from umbrella_b200 import seq_bench
    d = tempfile.mkdtemp(prefix=args.family + "_synth_")
    make = {"zedotar": seq_bench.zedotar_config, "kulisun": seq_bench.kulisun_config, "subivik": seq_bench.subivik_config}.get(args.family, seq_bench.radanex_config)
    json.dump(make(args.synthetic_width), open(os.path.join(d, "config.json"), "w"))
    config.update(model=d, synthetic=True)
engine = AutoEngine.from_config("cuda:0", **config)
engine.initialize()
vocab = engine.model.spec.vocab
g = torch.Generator().manual_seed(0)
prompts = [torch.randint(0, vocab, (max(1, args.prompt_len - 7 * i),), generator=g).tolist() for i in range(args.prompts)]
torch.cuda.synchronize()
t0 = time.time()
outs = engine.generate_batch(prompts, max_new_tokens=args.max_new_tokens)
torch.cuda.synchronize()
dt = time.time() - t0
n = sum(len(o) for o in outs)
print(json.dumps({"requests": len(outs), "generated_tokens": n, "seconds": round(dt, 3), "tokens_per_second": round(n / dt, 1)}))
print("first request:", outs[0][:16])
