"""Baseline TriMul submission: the straightforward PyTorch formulation in the input's dtype.
``trimul-baseline`` times it through the evaluation driver to obtain ``baseline_ns``, the
denominator of the speed term of the TriMul reward."""
import torch
import torch.nn.functional as F


def custom_kernel(data):
    x, mask, w, cfg = data
    xn = F.layer_norm(x, (cfg["dim"],), w["norm.weight"], w["norm.bias"])
    m = mask.unsqueeze(-1)
    left = F.linear(xn, w["left_proj.weight"]) * m * torch.sigmoid(F.linear(xn, w["left_gate.weight"]))
    right = F.linear(xn, w["right_proj.weight"]) * m * torch.sigmoid(F.linear(xn, w["right_gate.weight"]))
    gate = torch.sigmoid(F.linear(xn, w["out_gate.weight"]))
    out = torch.einsum("bikd,bjkd->bijd", left, right)
    out = F.layer_norm(out, (cfg["hidden_dim"],), w["to_out_norm.weight"], w["to_out_norm.bias"])
    return F.linear(out * gate, w["to_out.weight"])
