"""Times the reference's own modules (staged under baseline/_ref by stage_ref.py) on the current GPU.

    python baseline/ref_gpu_step.py B D STEPS

Runs MemoryEfficientCLIPLoss(temperature=0.07, normalized_inputs=True) forward + backward on fp32
row-normalised N(0,1) features (the reference's Triton backward takes fp32 only: its tl.dot mixes an
fp32 coefficient tile with the input dtype) and prints one JSON line.  Run as a child process by
bench.py, outside every timed region; nothing of this repository's package is imported here.
"""
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "_ref"))


def main():
    b, d, steps = int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3])
    import torch
    from clip_loss import MemoryEfficientCLIPLoss      # the reference's file, not this repository's package
    g = torch.Generator().manual_seed(0)
    x = torch.nn.functional.normalize(torch.randn(b, d, generator=g), dim=1).cuda().requires_grad_(True)
    y = torch.nn.functional.normalize(torch.randn(b, d, generator=g), dim=1).cuda().requires_grad_(True)
    mod = MemoryEfficientCLIPLoss(temperature=0.07, normalized_inputs=True)

    def step():
        x.grad = None
        y.grad = None
        loss = mod(x, y)
        loss.backward()
        return loss

    step()                                              # JIT compilation + first launch
    torch.cuda.synchronize()
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    marks[0].record()
    for i in range(steps):
        loss = step()
        marks[i + 1].record()
    torch.cuda.synchronize()
    ms = marks[0].elapsed_time(marks[steps]) / steps
    print(json.dumps({"ms_per_step": ms, "tflops": 8.0 * b * b * d / (ms / 1e3) / 1e12, "steps": steps,
                      "batch": b, "feature_dim": d, "dtype": "f32(tf32 tl.dot)", "loss": float(loss)}))


if __name__ == "__main__":
    main()
