"""Generate tests/golden/ref_fakequant.npz from the REFERENCE's own torch code.

The reference (vitali87/quadbit) keeps its fake-quant / packing functions as closures
inside Modal entry points (`import modal` at module level, device hard-coded to CUDA),
so the files cannot be imported. This script parses the reference sources with `ast`,
lifts the named closure definitions and table assignments out of their enclosing
function UNCHANGED, executes them with `dev = torch.device("cpu")`, and stores inputs
and outputs as a compressed .npz. The committed .npz is what the test-suite reads; the
reference tree is only needed when regenerating:

    python tests/golden/make_golden.py /path/to/quadbit

Inputs follow the reference's own test recipe (`torch.randn(out,in)*0.02`, `torch.randn`
activations, harness/verify_sparse_2lvl.py:188-193) plus rows scaled over many decades to
exercise the scale encoder's clamps. fp32 random inputs have no importance ties, which the
script asserts (the reference's tie order is unspecified).
"""
from __future__ import annotations

import ast
import sys
from pathlib import Path

import numpy as np
import torch
import torch.nn.functional as F


def lift(path: Path, names: set[str], inside: str = "run", extra_ns: dict | None = None) -> dict:
    """Execute, on CPU, the nested defs/assignments called `names` found in the body of the
    top-level function `inside` of `path`."""
    tree = ast.parse(path.read_text())
    scope = next(n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == inside)
    picked = []
    for node in scope.body:
        if isinstance(node, ast.FunctionDef) and node.name in names:
            picked.append(node)
        elif isinstance(node, ast.Assign):
            tgt = set()
            for t in node.targets:
                for n in ast.walk(t):
                    if isinstance(n, ast.Name):
                        tgt.add(n.id)
            if tgt & names:
                picked.append(node)
    picked.sort(key=lambda n: n.lineno)
    ns = {"torch": torch, "F": F, "dev": torch.device("cpu")}
    ns.update(extra_ns or {})
    mod = ast.Module(body=picked, type_ignores=[])
    exec(compile(mod, str(path), "exec"), ns)
    return ns


def lift_top(path: Path, names: set[str]) -> dict:
    """Same for module-level defs / assignments."""
    tree = ast.parse(path.read_text())
    picked = []
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name in names:
            picked.append(node)
        elif isinstance(node, ast.Assign) and any(isinstance(t, ast.Name) and t.id in names for t in node.targets):
            picked.append(node)
    ns = {"torch": torch}
    exec(compile(ast.Module(body=picked, type_ignores=[]), str(path), "exec"), ns)
    return ns


def main(ref_root: str) -> None:
    ref = Path(ref_root)
    tables = {"FP4", "BND", "_cc", "_c", "_e", "_m", "UE4M3"}
    v = lift(ref / "harness/verify_sparse_2lvl.py",
             tables | {"q_fp4", "enc_ue4m3_t", "pair24", "sparse_fp4_dequant_2lvl", "act_2lvl_deq_p32",
                       "pack_weight_2lvl", "deq_from_kernel_act_2lvl"})
    r = lift(ref / "harness/recovery_worth.py",
             tables | {"q_fp4", "enc_ue4m3_t", "act_fp4_dequant", "dense_fp4_dequant"})
    d = lift(ref / "harness/dense_e2e.py", tables | {"quant_fp4", "enc_ue4m3", "nvfp4_pack"})
    m = lift(ref / "harness/fused_moe.py", tables | {"q_fp4", "enc", "pack", "build_routing", "_BN"})
    # the plugin's packer takes activation column norms (Wanda importance) as a second argument
    pl = lift(ref / "harness/qb_vllm_plugin/qb_sm120_plugin.py", {"fp4", "bnd", "cc", "e_", "m_", "ue4m3", "q_fp4", "enc", "pack"},
              inside="_load_sparse_moe",
              extra_ns={"_FP4_VALS": [0, .5, 1, 1.5, 2, 3, 4, 6, 0, -.5, -1, -1.5, -2, -3, -4, -6]})

    g = torch.Generator().manual_seed(0)
    out = {}

    # primitives
    s = torch.cat([torch.tensor([0.0, 1e-30, 2.0 ** -10, 2.0 ** -9, 0.0019, 0.00195, 0.0137, 1.0, 1.0625, 1.9375,
                                 1.97, 447.0, 448.0, 464.0, 479.9, 480.0, 1e4]),
                   torch.exp(torch.empty(4000).uniform_(-25, 8, generator=g))]).float()
    out["enc_in"] = s.numpy()
    out["enc_out"] = v["enc_ue4m3_t"](s).numpy().astype(np.uint8)
    q = torch.cat([torch.tensor([0, .25, .75, 1.25, 1.75, 2.5, 3.5, 5., 6., 7., -0.25, -.75, -2.5, -5., -100.]),
                   torch.empty(4000).uniform_(-7, 7, generator=g)]).float()
    out["q_in"] = q.numpy()
    out["q_out"] = v["q_fp4"](q).numpy().astype(np.uint8)

    # sparse weights (reference recipe + decade-scaled rows)
    W = torch.randn(128, 512, generator=g) * 0.02
    W[96:] *= torch.pow(10.0, torch.linspace(-9, 4, 32)).view(32, 1)
    imp = W.view(128, 64, 4, 2).abs().sum(-1).sort(-1, descending=True).values
    assert int((imp[..., 1] == imp[..., 2]).sum()) == 0, "importance tie in golden input"
    Ac, meta, scaleA, gA, ks = v["pack_weight_2lvl"](W)
    out.update(sw=W.numpy(), sw_Ac=Ac.numpy(), sw_meta=meta.numpy(), sw_scaleA=scaleA.numpy(), sw_gA=gA.numpy(),
               sw_deq=v["sparse_fp4_dequant_2lvl"](W).numpy())
    pk = m["pack"](W.to(torch.bfloat16))       # MoE packer takes bf16 weights, has the zero-block guard
    Wb = W.to(torch.bfloat16).float()
    impb = Wb.view(128, 64, 4, 2).abs().sum(-1).sort(-1, descending=True).values
    out["swb_tiefree"] = (impb[..., 1] != impb[..., 2]).view(128, 4, 16).permute(1, 0, 2).numpy()  # [ks,out,16]
    out.update(swb_Ac=pk[0].numpy(), swb_meta=pk[1].numpy(), swb_scaleA=pk[2].numpy(), swb_gA=pk[3].numpy())

    # activations
    x = torch.randn(48, 512, generator=g)
    x[40:] *= torch.pow(10.0, torch.linspace(-6, 3, 8)).view(8, 1)
    out.update(ax=x.numpy(), ax_deq32=v["act_2lvl_deq_p32"](x).numpy(), ax_deq16=r["act_fp4_dequant"](x).numpy())

    # dense weights
    Wd = torch.randn(64, 512, generator=g) * 0.02
    Wd[48:] *= torch.pow(10.0, torch.linspace(-9, 4, 16)).view(16, 1)
    Ab, SFA, gAd = d["nvfp4_pack"](Wd)
    out.update(dw=Wd.numpy(), dw_Ab=Ab.numpy(), dw_SFA=SFA.numpy(), dw_gA=gAd.numpy(),
               dw_deq=r["dense_fp4_dequant"](Wd).numpy())

    # linear (fake-quant) results
    out["lin_sparse"] = F.linear(v["act_2lvl_deq_p32"](x), v["sparse_fp4_dequant_2lvl"](W)).numpy()
    out["lin_dense"] = F.linear(r["act_fp4_dequant"](x), r["dense_fp4_dequant"](Wd)).numpy()

    # MoE routing helper
    assign = torch.randint(0, 8, (300,), generator=g)
    src, eblk, r_pad = m["build_routing"](assign, 8)
    out.update(rt_assign=assign.numpy(), rt_src=src.numpy(), rt_eblk=eblk.numpy(), rt_rpad=np.int64(r_pad),
               rt_bn=np.int64(m["_BN"]))

    # activation-aware pair selection (drawn last so that every array above keeps its values)
    Ww = torch.randn(64, 256, generator=g) * 0.02
    cn = torch.exp(torch.empty(256).uniform_(-2, 2, generator=g))
    impw = (Ww.view(64, 32, 4, 2).abs() * cn.view(1, 32, 4, 2)).sum(-1).sort(-1, descending=True).values
    assert int((impw[..., 1] == impw[..., 2]).sum()) == 0, "importance tie in the column-norm golden input"
    pw = pl["pack"](Ww, cn)
    pz = pl["pack"](Ww, torch.zeros(256))          # all-zero norms: magnitude fallback
    out.update(ww=Ww.numpy(), ww_cn=cn.numpy(), ww_Ac=pw[0].numpy(), ww_meta=pw[1].numpy(), ww_scaleA=pw[2].numpy(),
               ww_gA=pw[3].numpy(), wz_Ac=pz[0].numpy(), wz_meta=pz[1].numpy())

    # checkpoint block formats (drawn after everything else)
    plugin = ref / "harness/qb_vllm_plugin/qb_sm120_plugin.py"
    mx = lift(plugin, {"fp4", "_mxfp4_dequant"}, inside="_install_gptoss_moe",
              extra_ns={"_FP4_VALS": [0, .5, 1, 1.5, 2, 3, 4, 6, 0, -.5, -1, -1.5, -2, -3, -4, -6]})
    nv = lift_top(plugin, {"_FP4_VALS", "_FP4_LUT_CACHE", "_dequant_nvfp4_expert"})
    cw = torch.randint(0, 256, (24, 96), generator=g, dtype=torch.int32).to(torch.uint8)            # [out, in/2], in = 192
    cs8 = torch.randint(100, 150, (24, 6), generator=g, dtype=torch.int32).to(torch.uint8)          # e8m0, one per 32
    cs4 = torch.randint(0, 0x7f, (24, 12), generator=g, dtype=torch.int32).to(torch.uint8)          # e4m3fn bytes, one per 16
    cs4[0, :3] = torch.tensor([0, 1, 0x7e], dtype=torch.uint8)                                      # zero, smallest subnormal, 448
    s2 = 0.01234
    out.update(ck_w=cw.numpy(), ck_s8=cs8.numpy(), ck_s4=cs4.numpy(), ck_s2=np.float32(s2),
               ck_mx=mx["_mxfp4_dequant"](cw, cs8).view(torch.int16).numpy(),
               ck_nv=nv["_dequant_nvfp4_expert"](cw, cs4.view(torch.float8_e4m3fn), torch.tensor(s2)).view(torch.int16).numpy())

    # single-level per-32 activation fake-quant, the torch twin of the legacy quant_act kernel ("kernel-MATCHED STE":
    # bf16 pre-round + no-denormal scale encode, harness/probe_ste_kernel.py:98-103); reuses x, draws nothing
    ps = lift(ref / "harness/probe_ste_kernel.py", tables | {"q_fp4", "enc_ue4m3_t", "act_fp4_dequant_km"})
    out["ax_deq32_1lvl"] = ps["act_fp4_dequant_km"](x).numpy()

    dst = Path(__file__).with_name("ref_fakequant.npz")
    np.savez_compressed(dst, **out)
    print(f"wrote {dst} ({dst.stat().st_size/1024:.0f} KiB, {len(out)} arrays)")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/quadbit")
    main(sys.argv[1])
