"""Copy-engine bandwidth between two GPUs of one process: one direction alone, then
both directions at once (the denominator of the link rooflines is the first figure).

    python -m stdml_collective_experimental_b200.benchmarks.link_copy

1 GiB per copy, 10 copies per direction, CUDA events on the copying streams."""
import torch, json
n = 1 << 30
a0 = torch.empty(n, dtype=torch.uint8, device="cuda:0"); b0 = torch.empty(n, dtype=torch.uint8, device="cuda:0")
a1 = torch.empty(n, dtype=torch.uint8, device="cuda:1"); b1 = torch.empty(n, dtype=torch.uint8, device="cuda:1")
s0 = torch.cuda.Stream("cuda:0"); s1 = torch.cuda.Stream("cuda:1")
def run(both, iters=10):
    for dev in (0, 1): torch.cuda.synchronize(dev)
    e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
    f0 = torch.cuda.Event(enable_timing=True); f1 = torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(s0):
        e0.record(s0)
        for _ in range(iters): b0.copy_(a1, non_blocking=True)   # dev0 pulls from dev1
        e1.record(s0)
    if both:
        with torch.cuda.stream(s1):
            f0.record(s1)
            for _ in range(iters): b1.copy_(a0, non_blocking=True)   # dev1 pulls from dev0
            f1.record(s1)
    for dev in (0, 1): torch.cuda.synchronize(dev)
    out = {"dir01_gb_s": n * iters / (e0.elapsed_time(e1) * 1e-3) / 1e9}
    if both: out["dir10_gb_s"] = n * iters / (f0.elapsed_time(f1) * 1e-3) / 1e9
    return out
run(True, 2)
print(json.dumps({"one_direction": run(False), "both_directions": run(True)}))
