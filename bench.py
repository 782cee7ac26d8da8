r"""
Headline benchmark: expert-parallel MoE MLP layer, forward + backward, tokens/s.

Config (fixed): bf16, 4096 tokens per GPU, d_model 1024, d_hidden 4096, 2 experts per GPU,
NaiveGate top-2 with a random-init gate, GELU; synthetic N(0,1) inputs, random-init weights.
One step = forward, backward, gradient all-reduce of the replicated (gate) parameters when
N > 1, and a fused Adam step on all parameters.  Weak scaling: per-GPU work is fixed.

    python bench.py --gpus 1 --steps 20 --warmup 5            # this framework
    python bench.py --impl reference ...                      # unmodified FastMoE from baseline/_ref
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N ...                 # N > 1

Timing: the GPU is first brought to its working clocks by one second of the step itself (both
arms alike; parameters and optimizer state are restored afterwards, and these steps are reported
as pre-heat, not as warm-up), then exactly W warm-up steps run (W >= 3), then every
one of the K timed steps is bracketed by CUDA events on the launching stream; an L2 flush (a
256 MiB fill) runs between steps outside the events; the K per-step times are summed per rank
and the maximum over ranks is reported.  SM clocks and throttle reasons are sampled with
nvidia-smi from the pre-heat to the end of the end-to-end region.  The end-to-end number re-runs the K
steps through the same public call with, per step, a host-to-device copy of the inputs from
pinned memory and a device-to-host read of the loss inside the timed region.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
PREHEAT_S = 1.0

METRIC = "moe_fwd_bwd_tokens_per_s"

# The headline config and the skewed, capacity-limited config of the baseline definition.
CONFIGS = {
    "ep_mlp": dict(tokens=4096, d_model=1024, d_hidden=4096, experts=2, top_k=2, gate="NaiveGate",
                   zipf=0.0, label="FMoETransformerMLP (EP MoE MLP layer, NaiveGate top-2, GELU)"),
    "skewed": dict(tokens=8192, d_model=2048, d_hidden=8192, experts=8, top_k=2, gate="GShardGate",
                   zipf=1.2, label="FMoETransformerMLP (GShardGate top-2, capacity 1.2, Zipf(1.2) gate bias, GELU)"),
}
# Whole language models (pure torch.nn around the MoE layer class of the arm being measured, so
# that both arms run the same dense code and differ only in the MoE implementation).
CONFIGS.update({
    "txl": dict(kind="lm", layers=12, d_model=512, heads=8, d_hidden=2048, experts=8, top_k=2,
                gate="NaiveGate", vocab=256, seq=512, mem=512, batch=22, zipf=0.0, shadow=False,
                label="Transformer-XL-style MoE LM (12 layers, d 512, 8 heads, every FFN an "
                      "FMoETransformerMLP with 8 experts/GPU, top-2 NaiveGate, seq 512 + mem 512)"),
    "gpt": dict(kind="lm", layers=24, d_model=1024, heads=16, d_hidden=4096, experts=2, top_k=1,
                gate="SwitchGate", vocab=50257, seq=1024, mem=0, batch=8, zipf=1.2, shadow=False,
                label="GPT with every FFN an FMoETransformerMLP (24 layers, h 1024, 16 heads, FFN 4096, "
                      "2 experts/GPU, SwitchGate top-1, Zipf(1.2) gate bias)"),
})
CONFIGS["gpt_shadow"] = dict(CONFIGS["gpt"], shadow=True,
                             label=CONFIGS["gpt"]["label"] + ", FasterMoE smart schedule + shadow experts on")
for _name in ("ep_mlp", "skewed"):
    CONFIGS[_name]["kind"] = "layer"
TOKENS_PER_GPU = D_MODEL = D_HIDDEN = EXPERTS_PER_GPU = TOP_K = None
CFG = None
GATE_NAME = ZIPF = MODEL_LABEL = None


def select_config(name):
    global TOKENS_PER_GPU, D_MODEL, D_HIDDEN, EXPERTS_PER_GPU, TOP_K, GATE_NAME, ZIPF, MODEL_LABEL, CFG
    c = CONFIGS[name]
    CFG = c
    if c["kind"] == "lm":
        c["tokens"] = c["batch"] * c["seq"]
        if c["shadow"]:
            # read by both implementations (the reference decides at import time)
            os.environ["FMOE_FASTER_SCHEDULE_ENABLE"] = "1"
            os.environ["FMOE_FASTER_SHADOW_ENABLE"] = "1"
    TOKENS_PER_GPU, D_MODEL, D_HIDDEN = c["tokens"], c["d_model"], c["d_hidden"]
    EXPERTS_PER_GPU, TOP_K, GATE_NAME, ZIPF, MODEL_LABEL = c["experts"], c["top_k"], c["gate"], c["zipf"], c["label"]


def skew_gate(layer, world):
    r"""Gate bias -s*log(rank of expert): expert popularity follows a Zipf law (random-init weights)."""
    import torch
    if ZIPF > 0:
        tot = EXPERTS_PER_GPU * world
        bias = -ZIPF * torch.log(torch.arange(1, tot + 1, dtype=torch.float32))
        with torch.no_grad():
            layer.gate.gate.weight.mul_(0.1)
            layer.gate.gate.bias.copy_(bias)


def kept_slot_fraction(layer, x):
    r"""Share of the top-k slots of one batch that survive the gate's capacity limit (1.0 for
    gates that drop nothing).  Run once, outside every timed region."""
    import torch
    try:
        with torch.no_grad():
            idx = layer.gate(x)[0]
        return float((idx >= 0).float().mean())
    except Exception:  # pylint: disable=broad-except
        return 1.0


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="ep_mlp", choices=sorted(CONFIGS))
    return ap.parse_args()


def emit(obj):
    print(json.dumps(obj), flush=True)


def give_up_reference(reason, rank, world):
    r"""The reference arm could not run: say why in the one JSON line, then leave quietly (process
    group closed first, so that the JSON line stays the last line of the output)."""
    if rank == 0:
        emit({"impl": "reference", "unavailable": reason[:400]})
    sys.stdout.flush()
    os._exit(0)  # pylint: disable=protected-access


# ------------------------------------------------------------------------------ clocks
class ClockSampler:
    r"""Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu_index), "--query-gpu=" + self.QUERY,
                 "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 8:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------ LM around the MoE layer
def make_lm(moe_cls, gate_cls, world, cfg):
    r"""A decoder-only LM in plain torch.nn; ``moe_cls`` / ``gate_cls`` come from the implementation
    under test.  With ``mem > 0`` every layer attends over [previous segment's hidden states;
    current segment] (Transformer-XL recurrence; learned absolute positions instead of the
    relative encoding, the same in both arms)."""
    import torch
    import torch.nn as nn
    import torch.nn.functional as F

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            d = cfg["d_model"]
            self.ln1, self.ln2 = nn.LayerNorm(d), nn.LayerNorm(d)
            self.qkv, self.proj = nn.Linear(d, 3 * d), nn.Linear(d, d)
            self.moe = moe_cls(num_expert=cfg["experts"], d_model=d, d_hidden=cfg["d_hidden"],
                               world_size=world, top_k=cfg["top_k"], gate=gate_cls,
                               activation=nn.GELU())

        def forward(self, x, mem):
            b, s, d = x.shape
            h = self.ln1(x)
            ctx = h if mem is None else torch.cat([mem, h], 1)
            q = self.qkv(h)[..., :d]
            kv = self.qkv(ctx)[..., d:]
            nh = cfg["heads"]
            q = q.view(b, s, nh, d // nh).transpose(1, 2)
            k, v = kv.view(b, ctx.shape[1], 2, nh, d // nh).permute(2, 0, 3, 1, 4)
            if mem is None:
                att = F.scaled_dot_product_attention(q, k, v, is_causal=True)
            else:
                m = ctx.shape[1] - s
                mask = torch.ones(s, ctx.shape[1], dtype=torch.bool, device=x.device).tril(m)
                att = F.scaled_dot_product_attention(q, k, v, attn_mask=mask)
            x = x + self.proj(att.transpose(1, 2).reshape(b, s, d))
            return x + self.moe(self.ln2(x)), h.detach()

    class LM(nn.Module):
        def __init__(self):
            super().__init__()
            d = cfg["d_model"]
            self.emb = nn.Embedding(cfg["vocab"], d)
            self.pos = nn.Embedding(cfg["seq"], d)
            self.blocks = nn.ModuleList([Block() for _ in range(cfg["layers"])])
            self.ln = nn.LayerNorm(d)
            self.head = nn.Linear(d, cfg["vocab"], bias=False)
            self.mems = None

        def forward(self, tokens):
            b, s = tokens.shape
            x = self.emb(tokens) + self.pos(torch.arange(s, device=tokens.device))
            new_mems = []
            for i, blk in enumerate(self.blocks):
                mem = self.mems[i] if (cfg["mem"] > 0 and self.mems is not None) else None
                x, h = blk(x, mem)
                new_mems.append(h[:, -cfg["mem"]:] if cfg["mem"] > 0 else None)
            if cfg["mem"] > 0:
                self.mems = new_mems
            logits = self.head(self.ln(x))
            loss = F.cross_entropy(logits.view(-1, logits.shape[-1]).float(), tokens.view(-1))
            for blk in self.blocks:
                if getattr(blk.moe.gate, "has_loss", False):
                    loss = loss + blk.moe.gate.get_loss().sum().float()
            return loss

    return LM()


def finish_lm(model, world, cfg, device, ddp_cls):
    import torch
    if cfg["zipf"] > 0:
        tot = cfg["experts"] * world
        bias = -cfg["zipf"] * torch.log(torch.arange(1, tot + 1, dtype=torch.float32))
        with torch.no_grad():
            for blk in model.blocks:
                blk.moe.gate.gate.weight.mul_(0.1)
                blk.moe.gate.gate.bias.copy_(bias)
    model = model.to(device).to(torch.bfloat16)
    wrapped = ddp_cls(model) if world > 1 else model
    return model, wrapped


# ------------------------------------------------------------------------------ the two arms
def build_ours(rank, world, device):
    import torch
    sys.path.insert(0, ROOT)
    from fastmoe_b200 import DistributedGroupedDataParallel, FMoETransformerMLP
    from fastmoe_b200 import gates
    from fastmoe_b200.ops import native
    native.get()  # fail loudly if the extension is missing
    torch.manual_seed(1234 + rank)
    if CFG["kind"] == "lm":
        lm = make_lm(FMoETransformerMLP, getattr(gates, GATE_NAME), world, CFG)
        lm, model = finish_lm(lm, world, CFG, device, DistributedGroupedDataParallel)
        return lm, model, (lambda: native.get().launch_count())
    layer = FMoETransformerMLP(num_expert=EXPERTS_PER_GPU, d_model=D_MODEL, d_hidden=D_HIDDEN,
                               world_size=world, top_k=TOP_K, gate=getattr(gates, GATE_NAME),
                               activation=torch.nn.GELU())
    skew_gate(layer, world)
    layer = layer.to(device).to(torch.bfloat16)
    model = layer
    if world > 1:
        model = DistributedGroupedDataParallel(layer)
    return layer, model, (lambda: native.get().launch_count())


def build_reference(rank, world, device):
    import torch
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    shim_dir = os.path.join(ROOT, "baseline", "shims")
    # The reference imports `tree` (dm-tree), which is not installed: a small pure-python
    # stand-in lives in baseline/shims.  Nothing of this repository's package is imported.
    sys.path.insert(0, shim_dir)
    sys.path.insert(0, ref_dir)
    from fmoe import FMoETransformerMLP  # noqa: E402  (the reference's own package)
    from fmoe.distributed import DistributedGroupedDataParallel
    from fmoe import gates
    assert os.path.realpath(sys.modules["fmoe"].__file__).startswith(os.path.realpath(ref_dir))
    torch.manual_seed(1234 + rank)
    if CFG["kind"] == "lm":
        lm = make_lm(FMoETransformerMLP, getattr(gates, GATE_NAME), world, CFG)
        lm, model = finish_lm(lm, world, CFG, device, DistributedGroupedDataParallel)
        return lm, model, (lambda: 0)
    layer = FMoETransformerMLP(num_expert=EXPERTS_PER_GPU, d_model=D_MODEL, d_hidden=D_HIDDEN,
                               world_size=world, top_k=TOP_K, gate=getattr(gates, GATE_NAME),
                               activation=torch.nn.GELU())
    skew_gate(layer, world)
    layer = layer.to(device).to(torch.bfloat16)
    model = layer
    if world > 1:
        model = DistributedGroupedDataParallel(layer)
    return layer, model, (lambda: 0)


def main():
    args = parse_args()
    select_config(args.config)
    if args.impl == "reference" and not os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "fmoe")):
        emit({"impl": "reference", "unavailable": "baseline/_ref is not installed"})
        return

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run for --gpus > 1")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)

    try:
        build = build_reference if args.impl == "reference" else build_ours
        layer, model, launch_counter = build(rank, world, device)
    except Exception as exc:  # pylint: disable=broad-except
        if args.impl == "reference":
            give_up_reference("reference failed to start: %r" % (exc,), rank, world)
        raise

    is_lm = CFG["kind"] == "lm"
    # The layer configs replay the step from a CUDA graph (the fused path never reads a count on
    # the host); whole models run eagerly: their gates (capacity limits, shadow policy) and the
    # recurrence memory are not capture-safe in general.
    graphed = (args.impl == "ours" and not is_lm
               and os.environ.get("FMOE_BENCH_GRAPH", "1") == "1")
    overlap = (args.impl == "ours" and world > 1 and not is_lm
               and os.environ.get("FMOE_BENCH_OVERLAP", "1") == "1")
    if overlap:
        # Same Adam over the same parameters, as two optimizer objects: the expert parameters
        # need no gradient reduction, so their update runs while the gate gradients are being
        # all-reduced on the wrapper's side stream.
        local_params = [p for p in layer.parameters() if getattr(p, "dp_comm", "dp") == "none"]
        local_ids = {id(p) for p in local_params}
        synced_params = [p for p in layer.parameters() if id(p) not in local_ids]
        opt_local = torch.optim.Adam(local_params, lr=1e-4, fused=True, capturable=graphed)
        opt = torch.optim.Adam(synced_params, lr=1e-4, fused=True, capturable=graphed)
    else:
        opt_local = None
        opt = torch.optim.Adam(layer.parameters(), lr=1e-4, fused=True, capturable=graphed)
    n_inputs = 4
    gen = torch.Generator(device="cpu").manual_seed(99 + rank)
    if is_lm:
        host_inputs = [torch.randint(0, CFG["vocab"], (CFG["batch"], CFG["seq"]), generator=gen).pin_memory()
                       for _ in range(n_inputs)]
    else:
        host_inputs = [torch.randn(TOKENS_PER_GPU, D_MODEL, generator=gen).to(torch.bfloat16).pin_memory()
                       for _ in range(n_inputs)]
    dev_inputs = [h.to(device) for h in host_inputs]
    flush = torch.empty(256 * 1024 * 1024 // 4, dtype=torch.float32, device=device)

    def step(x):
        opt.zero_grad(set_to_none=True)
        if opt_local is not None:
            opt_local.zero_grad(set_to_none=True)
        if is_lm:
            loss = model(x)
        else:
            x = x.detach().requires_grad_(True)
            y = model(x)
            loss = y.sum()
            if layer.gate.has_loss:
                loss = loss + layer.gate.get_loss().sum().to(loss.dtype)
        loss.backward()
        if opt_local is not None:
            pending = model.allreduce_params(async_op=True)
            opt_local.step()
            pending.wait()
        elif world > 1:
            model.allreduce_params()
        opt.step()
        return loss

    if graphed:
        # The fused path has no host read, so the whole step is captured into one CUDA graph
        # through the framework's public helper; inputs are copied into its static buffer.
        from fastmoe_b200.utils.graph import GraphedStep
        eager_step = step
        count0 = launch_counter()
        stepper = GraphedStep(lambda x: eager_step(x), dev_inputs[0], warmup=3)
        # Replays do not pass through the Python bindings that count launches: one replay
        # launches what one eager step launched (3 warm-up runs + 1 captured run were counted).
        launches_per_step = (launch_counter() - count0) // 4

        def step(x):  # noqa: F811
            return stepper(x)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    # Clock ramp: the step itself, run for PREHEAT_S seconds (both arms alike), so that the timed
    # steps see the clocks of sustained training.  Parameters and optimizer state are put back
    # afterwards: the warm-up and the timed steps start from the random-init weights.
    def snapshot():
        tensors = [p.data for p in layer.parameters()]
        for o in (opt, opt_local):
            if o is not None:
                for st in o.state.values():
                    tensors.extend(v for v in st.values() if torch.is_tensor(v))
        return tensors, [t.clone() for t in tensors]

    preheat_steps = 0
    try:
        step(dev_inputs[0])          # creates the optimizer state that the snapshot covers
        torch.cuda.synchronize()
        live, saved = snapshot()
        t_heat = time.perf_counter()
        go_on = torch.ones(1, dtype=torch.int32, device=device)
        while int(go_on.item()) == 1:
            for _ in range(8):
                step(dev_inputs[preheat_steps % n_inputs])
                preheat_steps += 1
            torch.cuda.synchronize()
            # every rank must run the same number of steps: rank 0 decides when to stop
            go_on.fill_(1 if time.perf_counter() - t_heat < PREHEAT_S else 0)
            if world > 1:
                dist.broadcast(go_on, 0)
        with torch.no_grad():
            for t, s0 in zip(live, saved):
                t.copy_(s0)
        del saved
    except Exception as exc:  # pylint: disable=broad-except
        if rank == 0:
            sampler.stop()
        if args.impl == "reference":
            give_up_reference("reference step failed: %r" % (exc,), rank, world)
        raise

    warm_steps = max(args.warmup, 3)
    try:
        for i in range(warm_steps):
            step(dev_inputs[i % n_inputs])
        barrier()
    except Exception as exc:  # pylint: disable=broad-except
        if rank == 0:
            sampler.stop()
        if args.impl == "reference":
            give_up_reference("reference step failed: %r" % (exc,), rank, world)
        raise

    # ------------------------------------------------ device-timed region (inputs resident)
    launches_before = launch_counter()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    barrier()
    for i in range(args.steps):
        flush.fill_(float(i))
        starts[i].record()
        step(dev_inputs[i % n_inputs])
        ends[i].record()
    barrier()
    launches = launch_counter() - launches_before
    if graphed:
        launches = launches_per_step * args.steps
    step_ms = [s.elapsed_time(e) for s, e in zip(starts, ends)]
    dev_ms = sum(step_ms)

    # The same K steps without the CUDA graph (this framework only; extra key, not the headline).
    eager_ms = None
    if graphed:
        for i in range(3):
            eager_step(dev_inputs[i % n_inputs])
        barrier()
        eager_ms = 0.0
        for i in range(args.steps):
            flush.fill_(float(i))
            starts[i].record()
            eager_step(dev_inputs[i % n_inputs])
            ends[i].record()
        barrier()
        eager_ms = sum(s.elapsed_time(e) for s, e in zip(starts, ends))

    # ------------------------------------------------ end-to-end region (H2D inputs, D2H loss)
    # One timed region around all K steps.  Inside it, every step: the pinned host batch is
    # copied to the device (on a copy stream, up to three steps ahead of its use: a plain input
    # pipeline, the same for both arms), the step runs through the framework's public call,
    # and the loss is read back to the host (asynchronously into pinned memory; the host consumes
    # the value three steps later, so that a scheduling hiccup of one of the N host processes
    # does not stall the N GPUs that wait for each other on the device).  An L2 flush (160 MiB fill) also runs between the steps,
    # inside the region.
    main = torch.cuda.current_stream()
    copy_stream = torch.cuda.Stream()
    depth = 4   # input copies run up to `depth - 1` steps ahead; a loss is consumed `depth - 1` steps late
    stage = [torch.empty_like(dev_inputs[0]) for _ in range(depth)]
    ready = [torch.cuda.Event() for _ in range(depth)]
    consumed = [torch.cuda.Event() for _ in range(depth)]
    loss_pinned = [torch.zeros(1, dtype=torch.float32).pin_memory() for _ in range(depth)]
    loss_done = [torch.cuda.Event() for _ in range(depth)]
    small_flush = flush[:160 * 1024 * 1024 // 4]

    def issue_copy(i):
        j = i % depth
        with torch.cuda.stream(copy_stream):
            if i >= depth:
                copy_stream.wait_event(consumed[j])
            stage[j].copy_(host_inputs[i % n_inputs], non_blocking=True)
            ready[j].record(copy_stream)

    barrier()
    loss_host = 0.0
    s_ev = torch.cuda.Event(enable_timing=True)
    e_ev = torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    s_ev.record()
    for i in range(min(depth - 1, args.steps)):
        issue_copy(i)
    for i in range(args.steps):
        if i + depth - 1 < args.steps:
            issue_copy(i + depth - 1)
        small_flush.fill_(float(i))
        main.wait_event(ready[i % depth])
        loss = stepper(stage[i % depth]) if graphed else step(stage[i % depth])
        consumed[i % depth].record(main)
        loss_pinned[i % depth].copy_(loss.detach().float().reshape(1), non_blocking=True)
        loss_done[i % depth].record(main)
        if i >= depth - 1:
            # the result of an earlier step, on the host (every step's loss is read exactly once)
            loss_done[(i - depth + 1) % depth].synchronize()
            loss_host = float(loss_pinned[(i - depth + 1) % depth])
    for i in range(max(0, args.steps - depth + 1), args.steps):
        loss_done[i % depth].synchronize()
        loss_host = float(loss_pinned[i % depth])
    e_ev.record()
    torch.cuda.synchronize()
    wall = (time.perf_counter() - t0) * 1e3
    e2e_ms = max(s_ev.elapsed_time(e_ev), wall)
    barrier()

    clocks = sampler.stop() if rank == 0 else None

    kept = 1.0 if is_lm else kept_slot_fraction(layer, dev_inputs[0])
    times = torch.tensor([dev_ms, e2e_ms, eager_ms or 0.0, max(step_ms), -min(step_ms)],
                         dtype=torch.float64, device=device)
    sums = torch.tensor([kept], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        dist.all_reduce(sums)
    dev_ms, e2e_ms, eager_max = float(times[0]), float(times[1]), float(times[2])
    step_max, step_min = float(times[3]), -float(times[4])
    kept = float(sums[0]) / world

    if rank == 0:
        tokens = TOKENS_PER_GPU * world * args.steps
        value = tokens / (dev_ms / 1e3)
        e2e_value = tokens / (e2e_ms / 1e3)
        # Slots a capacity limit dropped do no work in the expert GEMMs: count the kept ones.
        flops_per_step = 3 * 2 * 2 * TOKENS_PER_GPU * TOP_K * kept * D_MODEL * D_HIDDEN * world
        if is_lm:
            # model FLOPs of fwd + bwd: attention projections and scores, top-k expert MLPs, LM head
            d, kv = D_MODEL, CFG["seq"] + CFG["mem"]
            per_token = CFG["layers"] * (8 * d * d + 4 * kv * d + TOP_K * 4 * d * D_HIDDEN) + 2 * d * CFG["vocab"]
            flops_per_step = 3 * per_token * TOKENS_PER_GPU * world
        out = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": warm_steps,
            "ms_per_step": dev_ms / args.steps, "ms_per_step_min": step_min,
            "ms_per_step_median": statistics.median(step_ms), "ms_per_step_max": step_max,
            "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16",
            "data": ("synthetic tokens, uniform over the vocabulary, random-init weights" if is_lm
                     else "synthetic N(0,1) inputs, random-init weights"),
            "impl": args.impl,
            "tflops": flops_per_step / (dev_ms / args.steps / 1e3) / 1e12,
            "config": {
                "name": args.config, "model": MODEL_LABEL,
                "tokens_per_gpu": TOKENS_PER_GPU, "global_batch": TOKENS_PER_GPU * world,
                "seq_len": CFG["seq"] if is_lm else 1, "d_model": D_MODEL, "d_hidden": D_HIDDEN,
                "experts_per_gpu": EXPERTS_PER_GPU, "top_k": TOP_K,
                "parallelism": "ep%d" % world,
                "step": ("fwd+bwd+grad-allreduce+fused-adam" if is_lm
                         else "fwd+bwd+gate-grad-allreduce+fused-adam"),
                "l2": "flushed between timed steps (256 MiB fill outside the per-step events; "
                      "in the end-to-end region a 160 MiB fill per step inside the region)",
            },
            "kept_slot_fraction": kept,
            "execution": {
                "cuda_graph": bool(graphed),
                "allreduce_overlap": ("gate-gradient all-reduce on a side stream, overlapped with the"
                                      " Adam update of the expert parameters (same Adam, two optimizer"
                                      " objects)") if overlap else "none",
                "preheat": "%.1f s of the same step before the warm-up steps (%d steps); parameters and"
                           " optimizer state restored afterwards" % (PREHEAT_S, preheat_steps),
                "eager_ms_per_step": (eager_max / args.steps) if graphed else None,
            },
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "tokens/s",
                    "h2d_bytes_per_step": host_inputs[0].numel() * host_inputs[0].element_size(),
                    "d2h_bytes_per_step": 4, "ms_per_step": e2e_ms / args.steps,
                    "last_loss": loss_host},
            "gpu_launches": int(launches),
        }
        emit(out)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
