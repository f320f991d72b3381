"""Set per-layer LIF thresholds of a random-init model so that each site fires at a target rate.

Random weights give arbitrary firing rates; the benchmark configurations ask for about 15 % on q/k/v
and 5 % on the MLP gate.  For every site, layer by layer, a scalar threshold is found by bisection on
the measured rate of the CUDA LIF kernel over a sample batch (dense causal attention, no paging),
then broadcast to the site's per-channel threshold vector.  A setup utility for synthetic models,
not part of the decode hot path.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .kernels import lif_multistep
from .modeling import SpikingQwenModel, rms_norm, rotate_half


def _fit(x: torch.Tensor, beta: torch.Tensor, target: float, lo: float = 1e-3, hi: float = 50.0, iters: int = 18):
    n = beta.numel()
    for _ in range(iters):
        mid = (lo * hi) ** 0.5
        th = torch.full((n,), mid, device=x.device)
        rate = lif_multistep(x, beta, th, out_dtype=torch.uint8).float().mean().item()
        if rate > target:
            lo = mid
        else:
            hi = mid
    return torch.full((n,), (lo * hi) ** 0.5, device=x.device)


@torch.no_grad()
def calibrate_thresholds(model: SpikingQwenModel, prompts: torch.Tensor, qkv_rate: float = 0.15,
                         gate_rate: float = 0.05) -> dict:
    """``prompts`` int64 ``[B, S]`` on the model's device.  Updates ``model.layers[*]['lif_*']`` in place
    and returns the measured rates per site kind."""
    c = model.config
    T, hq, hkv, d = c.T, c.num_attention_heads, c.num_key_value_heads, c.head_dim
    B, S = prompts.shape
    positions = torch.arange(S, device=model.device).repeat(B)
    cos, sin = model.rope(positions)
    cos, sin = cos[None, :, None, :], sin[None, :, None, :]
    h = F.embedding(prompts.reshape(-1), model.embed).unsqueeze(0).expand(T, B * S, -1).contiguous()
    rates = {"q": [], "k": [], "v": [], "gate": []}
    n_rot = hq + hkv
    for L in model.layers:
        x = rms_norm(h, L["ln1"], c.rms_norm_eps)
        qkv = F.linear(x, L["w_qkv"], L["b_qkv"])
        qk = qkv[..., : n_rot * d].unflatten(-1, (n_rot, d))
        qkv[..., : n_rot * d] = ((qk * cos) + (rotate_half(qk) * sin)).flatten(-2)
        parts = {"q": qkv[..., : hq * d].unflatten(-1, (hq, d)),
                 "k": qkv[..., hq * d:(hq + hkv) * d].unflatten(-1, (hkv, d)),
                 "v": qkv[..., (hq + hkv) * d:].unflatten(-1, (hkv, d))}
        spk = {}
        for name, cur in parts.items():
            beta = L[f"lif_{name}"][0]
            th = _fit(cur, beta, qkv_rate)
            L[f"lif_{name}"] = (beta, th)
            spk[name] = lif_multistep(cur, beta, th)  # [T, B*S, H, d]
            rates[name].append(spk[name].float().mean().item())
        to_bhsd = lambda s, H: s.view(T, B, S, H, d).permute(0, 1, 3, 2, 4).reshape(T * B, H, S, d)
        ctx = F.scaled_dot_product_attention(to_bhsd(spk["q"], hq), to_bhsd(spk["k"], hkv), to_bhsd(spk["v"], hkv),
                                             is_causal=True, enable_gqa=hq != hkv)
        ctx = ctx.view(T, B, hq, S, d).permute(0, 1, 3, 2, 4).reshape(T, B * S, hq * d)
        h = h + F.linear(ctx, L["w_o"])
        x = rms_norm(h, L["ln2"], c.rms_norm_eps)
        gu = F.linear(x, L["w_gate_up"])
        gate, up = gu[..., : c.intermediate_size], gu[..., c.intermediate_size:]
        beta = L["lif_gate"][0]
        th = _fit(gate, beta, gate_rate)
        L["lif_gate"] = (beta, th)
        gate_spk = lif_multistep(gate, beta, th)
        rates["gate"].append(gate_spk.float().mean().item())
        h = h + F.linear(gate_spk * up, L["w_down"])
    return {k: sum(v) / len(v) for k, v in rates.items()}
