"""MiniGPT-style decoder training step with every ``nn.Linear`` replaced by the AXS-6 Linear.

A caller of the hot path (the counterpart of the reference's ``examples/pretrain_gpt.py`` model and
of its MiniGPT benchmark): 12 pre-norm layers, d_model 1024, 16 heads, FFN 4096, sequence 1024,
vocabulary 32000, weights ~ N(0, 0.02), uniform-random tokens, batch 8 per GPU, AdamW, fp32 master
weights with bf16 compute.  Attention, layer norm, embedding, loss and optimiser are PyTorch;
all Linear layers (q, k, v, o, two FFN layers per block and the LM head) go through
``AXSLinearMixedPrecision`` (fake-quantise kernels + tcgen05 GEMMs).  With more than one rank the
replicas are wrapped in DistributedDataParallel (NCCL).
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from axs6_b200.unified.mixed_precision import AXSLinearMixedPrecision

LAYERS, D_MODEL, HEADS, FFN, SEQ, VOCAB, BATCH = 12, 1024, 16, 4096, 1024, 32000, 8


class _Bf16Linear(nn.Linear):
    """Plain bf16 tensor-core Linear with fp32 master weights (the un-quantised comparison)."""

    def forward(self, x):
        return F.linear(x.to(torch.bfloat16), self.weight.to(torch.bfloat16),
                        self.bias.to(torch.bfloat16) if self.bias is not None else None)


class Block(nn.Module):
    def __init__(self, linear):
        super().__init__()
        self.ln1, self.ln2 = nn.LayerNorm(D_MODEL), nn.LayerNorm(D_MODEL)
        self.q, self.k, self.v, self.o = (linear(D_MODEL, D_MODEL) for _ in range(4))
        self.fc1, self.fc2 = linear(D_MODEL, FFN), linear(FFN, D_MODEL)

    def forward(self, x):
        B, T, _ = x.shape
        h = self.ln1(x.float()).to(torch.bfloat16)
        q = self.q(h).view(B, T, HEADS, -1).transpose(1, 2)
        k = self.k(h).view(B, T, HEADS, -1).transpose(1, 2)
        v = self.v(h).view(B, T, HEADS, -1).transpose(1, 2)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B, T, D_MODEL)
        x = x + self.o(a)
        h = self.ln2(x.float()).to(torch.bfloat16)
        return x + self.fc2(F.gelu(self.fc1(h)))


class MiniGPT(nn.Module):
    def __init__(self, linear):
        super().__init__()
        self.tok = nn.Embedding(VOCAB, D_MODEL)
        self.pos = nn.Embedding(SEQ, D_MODEL)
        self.blocks = nn.ModuleList(Block(linear) for _ in range(LAYERS))
        self.ln_f = nn.LayerNorm(D_MODEL)
        self.head = linear(D_MODEL, VOCAB, bias=False)
        for m in self.modules():
            if isinstance(m, (nn.Linear, AXSLinearMixedPrecision)):
                nn.init.normal_(m.weight, 0.0, 0.02)
                if m.bias is not None:
                    nn.init.zeros_(m.bias)
            elif isinstance(m, nn.Embedding):
                nn.init.normal_(m.weight, 0.0, 0.02)

    def forward(self, tokens):
        B, T = tokens.shape
        x = (self.tok(tokens) + self.pos(torch.arange(T, device=tokens.device))).to(torch.bfloat16)
        for b in self.blocks:
            x = b(x)
        return self.head(self.ln_f(x.float()).to(torch.bfloat16))


def flops_per_step(batch: int = BATCH) -> float:
    tokens = batch * SEQ
    p_linear = LAYERS * (4 * D_MODEL * D_MODEL + 2 * D_MODEL * FFN) + D_MODEL * VOCAB
    return 6.0 * tokens * p_linear + 12.0 * LAYERS * batch * SEQ * SEQ * D_MODEL


def _graphed_step(dev, steps: int) -> dict:
    """The same AXS-6 training step captured ONCE in a CUDA graph (forward, loss, backward, fused
    AdamW) and replayed, which removes the host launch cost of about 1300 kernels per step (measured: the
    step is GPU-bound either way, 29 ms replayed against 31 ms eager).  The captured step starts with `philox_advance`, so every replay rounds the
    gradients with fresh draws although the host-side offsets are frozen in the graph."""
    from axs6_b200 import _lib, ops
    torch.manual_seed(1234)
    model = MiniGPT(lambda i, o, bias=True: AXSLinearMixedPrecision(i, o, bias=bias)).to(dev)
    opt = torch.optim.AdamW(model.parameters(), lr=3e-4, fused=True, capturable=True)
    g = torch.Generator(device=dev).manual_seed(7)
    tokens = torch.randint(0, VOCAB, (BATCH, SEQ), generator=g, device=dev)
    targets = torch.randint(0, VOCAB, (BATCH, SEQ), generator=g, device=dev)

    def body():
        ops.philox_advance(1 << 40)
        logits = model(tokens)
        loss = F.cross_entropy(logits.float().view(-1, VOCAB), targets.view(-1))
        loss.backward()
        opt.step()
        return loss

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    first = None
    with torch.cuda.stream(side):
        for _ in range(3):
            opt.zero_grad(set_to_none=True)
            loss = body()
            first = float(loss.detach()) if first is None else first
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    opt.zero_grad(set_to_none=True)
    l0 = _lib.launches()
    with torch.cuda.graph(graph):
        static_loss = body()
    captured = _lib.launches() - l0
    for _ in range(2):
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    res = {"ms_per_step": ms, "tokens_per_s": BATCH * SEQ / (ms * 1e-3), "TFLOPs": flops_per_step() / (ms * 1e-3) / 1e12,
           "loss_first": first, "loss_last": float(static_loss.detach()), "library_kernels_in_graph": captured}
    ops.philox_advance(0, reset=True)
    del graph, model, opt
    torch.cuda.empty_cache()
    return res


def run(args, rank: int, world: int, dev, steps: int = 8) -> dict:
    import torch.distributed as dist
    from axs6_b200 import _lib
    out = {}
    for name, linear in (("axs6", lambda i, o, bias=True: AXSLinearMixedPrecision(i, o, bias=bias)),
                         ("bf16_nn_linear", lambda i, o, bias=True: _Bf16Linear(i, o, bias=bias))):
        torch.manual_seed(1234)
        model = MiniGPT(linear).to(dev)
        net = model
        if world > 1:
            net = torch.nn.parallel.DistributedDataParallel(model, device_ids=[dev.index])
        opt = torch.optim.AdamW(net.parameters(), lr=3e-4, fused=True)
        g = torch.Generator(device=dev).manual_seed(7 + rank)
        tokens = torch.randint(0, VOCAB, (BATCH, SEQ), generator=g, device=dev)
        targets = torch.randint(0, VOCAB, (BATCH, SEQ), generator=g, device=dev)

        def step():
            opt.zero_grad(set_to_none=True)
            logits = net(tokens)
            loss = F.cross_entropy(logits.float().view(-1, VOCAB), targets.view(-1))
            loss.backward()
            opt.step()
            return loss

        losses = [float(step().detach()) for _ in range(3)]
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        l0 = _lib.launches()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            loss = step()
        e1.record()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item()) / steps
        out[name] = {"ms_per_step": ms, "tokens_per_s": world * BATCH * SEQ / (ms * 1e-3),
                     "TFLOPs": world * flops_per_step() / (ms * 1e-3) / 1e12,
                     "loss_first": losses[0], "loss_last": float(loss.detach()),
                     "library_kernel_launches_per_step": (_lib.launches() - l0) / steps}
        del model, net, opt
        torch.cuda.empty_cache()
    if world == 1:
        try:
            out["axs6_cuda_graph"] = _graphed_step(dev, steps)
        except Exception as e:            # reported, never fatal for the rest of the line
            out["axs6_cuda_graph"] = {"error": repr(e)}
    out["gemm_status"] = int(_lib.load().axs6_gemm_status())
    out["workload"] = (f"{LAYERS} layers, d_model {D_MODEL}, {HEADS} heads, FFN {FFN}, seq {SEQ}, vocab {VOCAB}, "
                       f"batch {BATCH} per GPU, AdamW, {world} GPU(s)")
    out["flops_per_step_per_gpu"] = flops_per_step()
    out["axs6_over_bf16_step_time"] = out["axs6"]["ms_per_step"] / out["bf16_nn_linear"]["ms_per_step"]
    if "ms_per_step" in out.get("axs6_cuda_graph", {}):
        out["axs6_cuda_graph_over_bf16_step_time"] = out["axs6_cuda_graph"]["ms_per_step"] / out["bf16_nn_linear"]["ms_per_step"]
    return out
