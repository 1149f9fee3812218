"""Child process that runs the unmodified reference on CPU and dumps what the parity tests compare against.

usage: python ref_oracle.py <reference dir> <out.pt> <json spec>
spec: {"name", "vocab", "env": {...}, "B", "T", "seed", "what": "model" | "instinct"}
The reference reads its switches from the environment at import time, hence the separate process."""
import json
import math
import os
import sys


def main():
    ref_dir, out, spec = os.path.abspath(sys.argv[1]), os.path.abspath(sys.argv[2]), json.loads(sys.argv[3])
    os.environ.update({"DEVICE": "cpu", "NO_COMPILE": "1"})
    os.environ.update({k: str(v) for k, v in spec.get("env", {}).items()})
    sys.path.insert(0, ref_dir)
    os.chdir(ref_dir)
    import torch
    if spec.get("stable_sort"):
        # The reference breaks ties in its slot choice with an unstable argsort, whose order on equal keys is an
        # implementation detail of the sort; the rule "smaller index first" makes the comparison well defined.
        plain = torch.Tensor.argsort

        def stable(self, dim=-1, descending=False, stable=True):
            return plain(self, dim=dim, descending=descending, stable=True)
        torch.Tensor.argsort = stable
    torch.manual_seed(spec.get("seed", 0))
    if spec["what"] == "model":
        import lm
        m = lm.build(spec["name"], spec["vocab"])
        m.train()
        sd = {k: v.clone() for k, v in m.state_dict().items()}
        if spec.get("freeze"):                            # move these experts of every bank layer into the frozen bank
            for b in m.heavy:
                b.learned.zero_()
                b.learned[spec["freeze"]] = True
            m.rebank(1000)
        g = torch.Generator().manual_seed(1)
        xy = torch.randint(0, spec["vocab"], (spec["B"], spec["T"] + 1), generator=g)
        outp, cost = m(xy[:, :-1])
        if hasattr(m, "train_loss"):
            loss = m.train_loss(outp, xy[:, 1:], True)
        else:
            loss = torch.nn.functional.cross_entropy(outp.float().view(-1, outp.shape[-1]), xy[:, 1:].reshape(-1))
        if not spec.get("no_backward"):
            (loss + 0.01 * cost.float()).backward()
        grads = {n: p.grad.clone() for n, p in m.named_parameters() if p.grad is not None}
        stats = {k: (v.detach().float().clone() if torch.is_tensor(v) else float(v)) for k, v in getattr(m, "stats", {}).items()}
        torch.save({"sd": sd, "xy": xy, "loss": loss.detach(), "cost": cost.detach().float(), "grads": grads,
                    "stats": stats, "tau": m.tau.clone() if hasattr(m, "tau") else None}, out)
    elif spec["what"] == "train":
        import argparse
        import numpy as np
        import fastloop
        a = argparse.Namespace(batch=spec["B"], micro=spec["B"], seq=spec["T"], lr=spec["lr"], read_cost=0.01,
                               steps=spec["total_steps"])
        tr = fastloop.Trainer(spec["name"], spec.get("stage", "ABX"), a)
        sd = {k: v.clone() for k, v in tr.model.state_dict().items()}
        if spec.get("wave_every"):                        # shorter wave period so that a few steps exercise the waves
            for b in tr.model.heavy:
                b.wave_every = int(spec["wave_every"])
        data = fastloop.GPUData(np.load(spec["tokens"]), seed=1)
        batches, losses = [], []
        for s_ in range(spec["steps"]):
            xy = data.batch(spec["B"], spec["T"])
            batches.append(xy.clone())
            losses.append(float(tr.step(xy, s_)))
        waves = {k: v.clone() for k, v in tr.model.state_dict().items()
                 if k.split(".")[-1] in ("learned", "err", "err_peak", "err_freeze", "move_peak", "last_move")}
        torch.save({"sd": sd, "batches": batches, "losses": losses, "waves": waves}, out)
    elif spec["what"] == "experience":
        import exp_opt
        torch.manual_seed(3)
        shapes = [tuple(s_) for s_ in spec["shapes"]]
        ps = [torch.nn.Parameter(torch.randn(*s_) * 0.1) for s_ in shapes]
        w0 = [p.detach().clone() for p in ps]
        opt = exp_opt.ExperienceOpt(ps, lr=spec["lr"], **spec.get("kw", {}))
        feed, ws = [], []
        for step in range(spec["steps"]):
            gs = [torch.randn(*s_) * 0.01 for s_ in shapes]
            sit = torch.randn(spec["d"]) + (3.0 if step % 3 == 0 else -3.0) * torch.ones(spec["d"])   # two kinds of batches
            loss = 3.0 + 0.4 * math.sin(step)
            for p, g_ in zip(ps, gs):
                p.grad = g_.clone()
            opt.step(torch.tensor(loss), sit)
            feed.append((gs, sit, loss))
            ws.append([p.detach().clone() for p in ps])
        torch.save({"w0": w0, "feed": feed, "ws": ws, "used": opt.used.clone()}, out)
    elif spec["what"] == "instinct":
        import exp_opt
        torch.manual_seed(3)
        shapes = [tuple(s) for s in spec["shapes"]]
        ps = [torch.nn.Parameter(torch.randn(*s) * 0.1) if len(s) else torch.nn.Parameter(torch.tensor(0.3)) for s in shapes]
        w0 = [p.detach().clone() for p in ps]
        opt = exp_opt.InstinctOptB(ps, lr=spec["lr"], **spec.get("kw", {}))
        gs, ws = [], []
        for step in range(spec["steps"]):
            g_step = [torch.randn(*s) * (0.01 * (1 + i)) if len(s) else torch.randn(()) * 0.01 for i, s in enumerate(shapes)]
            sit = torch.randn(spec["d"])
            opt.prepare(torch.tensor(3.0 - 0.1 * step), sit)
            for p, g in zip(ps, g_step):
                p.grad = g.clone()
                opt.update(p)
                p.grad = None
            opt.finish()
            gs.append((g_step, sit))
            ws.append([p.detach().clone() for p in ps])
        torch.save({"w0": w0, "gs": gs, "ws": ws, "gain": opt.gain.clone(), "rel": opt.rel.clone()}, out)


if __name__ == "__main__":
    main()
