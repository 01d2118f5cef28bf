"""A few training steps of a small MLP, with torch's own allocator ("native") or with the side-aware
pluggable allocator ("sideaware"): the losses must come out the same, whatever memory the tensors
live in.  Activations and weights are tens of MiB each, so most blocks take the side-aware path.
Runs in a process of its own (the allocator can only be replaced before the first CUDA allocation).
Prints one JSON line."""
import json
import sys

import torch


def main():
    mode = sys.argv[1] if len(sys.argv) > 1 else "sideaware"
    stats = None
    sa = None
    if mode == "sideaware":
        import l2_torch_alloc_b200 as pkg
        sa = pkg.sideaware_init()
    torch.manual_seed(1234)
    torch.backends.cuda.matmul.allow_tf32 = False
    width, batch, steps = 3072, 4096, 6
    model = torch.nn.Sequential(torch.nn.Linear(width, width), torch.nn.GELU(), torch.nn.Linear(width, width), torch.nn.GELU(),
                                torch.nn.Linear(width, width)).cuda()
    opt = torch.optim.AdamW(model.parameters(), lr=1e-3)
    gen = torch.Generator(device="cuda").manual_seed(99)
    losses = []
    for _ in range(steps):
        x = torch.randn(batch, width, device="cuda", generator=gen)
        y = torch.randn(batch, width, device="cuda", generator=gen)
        loss = torch.nn.functional.mse_loss(model(x), y)
        opt.zero_grad(set_to_none=True)
        loss.backward()
        opt.step()
        losses.append(float(loss.item()).hex())
    torch.cuda.synchronize()
    # steady state: the same step repeated, every allocation of a size seen before
    import time
    t0 = time.perf_counter()
    timed = 20
    for _ in range(timed):
        x = torch.randn(batch, width, device="cuda", generator=gen)
        y = torch.randn(batch, width, device="cuda", generator=gen)
        loss = torch.nn.functional.mse_loss(model(x), y)
        opt.zero_grad(set_to_none=True)
        loss.backward()
        opt.step()
    torch.cuda.synchronize()
    ms_per_step = (time.perf_counter() - t0) / timed * 1e3
    if sa is not None:
        stats = sa.stats()
    print("RESULT " + json.dumps({"mode": mode, "losses": losses, "ms_per_step": ms_per_step, "stats": stats,
                                  "errors": sa.error_count() if sa else 0}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
