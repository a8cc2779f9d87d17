"""One prefill and a few single-token steps of a Lepalorn of real layer shapes (random weights): the workload the ncu
captures of profiles/lepalorn_kernels.md were taken on.  python profiles/lepalorn_probe.py [size] [prompt_len] [steps]"""
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
for p in (str(ROOT), str(ROOT / "lit-llama-ja_b200")):
    sys.path.insert(0, p)
import torch

import bench_models as BM

size = sys.argv[1] if len(sys.argv) > 1 else "w1024"
T = int(sys.argv[2]) if len(sys.argv) > 2 else 2048
steps = int(sys.argv[3]) if len(sys.argv) > 3 else 4
dev = torch.device("cuda", 0)
s = dict(BM.SIZES[size], layers=2)
with torch.no_grad():
    m = BM.lepalorn_model(s, dev)
    m.use_step_graph = False            # every kernel of a step as a launch of its own
    idx = torch.randint(0, BM.VOCAB, (1, T + steps), device=dev)
    m(idx[:, :T], T + 64, torch.arange(T))
    for t in range(T, T + steps):
        m(idx[:, t:t + 1], T + 64, torch.arange(t, t + 1))
torch.cuda.synchronize()
print("ok")
