"""quantize(model, calib_data_loader, config): collect the nn.Linear layers of a model, build a SegmentLinear for
each, calibrate them through forward hooks on the float model and swap them in.

Same call, config schema and phase order as the reference's segquant/torch/quantization.py:259-425
(collect :24-50, create :53-108, trace :110-141, smooth :143-146, calibrate :147-179, alpha search :181-242,
replace :244-257): the result is the model with SegmentLinear modules in place of its linears, which
`torch.save(model)` / `torch.load(..., weights_only=False)` round-trips (the reference's on-disk form,
test/test_affine.py:36-51): int8 / e4m3 weights as [N, K] byte tensors, int4 weights packed two per byte --
[N, K/2] for K-segmented layers, (S, N/S * K/2) for N-segmented ones (segment_tensor_manager.py:56-80).

What is NOT here: the graph pattern detector (segquant/pattern_detector.py).  Which linears are segmented, and
which follow an activation (DualScale), is therefore given explicitly:

    seg_map     {layer name: {"seg_mode": "weight" | "input", "chunks": n} or {..., "chunksizes": [...]}}
    dual_scale  iterable of layer names whose input is the output of an activation function

A config that asks for `seglinear` without a seg_map raises instead of silently quantising unsegmented.
"""
import fnmatch
import uuid

import torch
from torch import nn

from ..config import default_quantize_config
from ..layers.SegmentLinear import SegmentLinear


def _val(v):
    """Config entries may be enum members (segquant_b200.config) or their string values (a parsed YAML file)."""
    return getattr(v, "value", v)


def _move_to_device(batch, device):
    if isinstance(batch, torch.Tensor):
        return batch.to(device)
    if isinstance(batch, (tuple, list)):
        return tuple(_move_to_device(b, device) for b in batch)
    if isinstance(batch, dict):
        return {k: _move_to_device(v, device) for k, v in batch.items()}
    return batch


def _get_all_linears(model, default, config):
    off = [k for k, v in config.items() if k != "default" and v.get("enable") is False]
    on = [k for k, v in config.items() if k != "default" and v.get("enable") is True]
    found = {}
    for name, module in model.named_modules():
        if not isinstance(module, nn.Linear):
            continue
        enable = default
        if any(fnmatch.fnmatch(name, p) for p in off):
            enable = False
        if any(fnmatch.fnmatch(name, p) for p in on):
            enable = True
        if enable:
            found[name] = module
    return found


def _layer_config(name, final_config):
    """The first pattern entry that matches the layer name, else "default" (quantization.py:65-69).  Keys a pattern
    entry leaves out are taken from "default" (the reference needs every pattern entry to be complete)."""
    for pattern, cfg in final_config.items():
        if pattern != "default" and fnmatch.fnmatch(name, pattern):
            return {**final_config["default"], **cfg}
    return final_config["default"]


def _create_linear(layer, layer_name, seg_cfg, final_config, dual_scale=False, device=None):
    cfg = _layer_config(layer_name, final_config)

    def split(key):
        d = dict(cfg[key])
        return _val(d.pop("type")), d

    real_quant = cfg["real_quant"]
    in_type, in_args = split("input_quant")
    w_type, w_args = split("weight_quant")
    opt_type, opt_args = split("opt")
    calib_type, calib_args = split("calib")
    has_bias = getattr(layer, "bias", None) is not None
    chunksizes = seg_cfg.get("chunksizes")
    return SegmentLinear(
        layer.in_features, layer.out_features, bias=has_bias, seg_mode=seg_cfg["seg_mode"],
        chunks=seg_cfg.get("chunks", len(chunksizes or [])), chunksizes=chunksizes,
        custom_weight_tensor=layer.weight.data, custom_bias_tensor=layer.bias.data if has_bias else None,
        input_quant_type=in_type, weight_quant_type=w_type,
        input_quant_args={"real_quant": real_quant, "dual_scale": dual_scale, **in_args},
        weight_quant_args={"real_quant": real_quant, **w_args},
        opt_type=opt_type, opt_kwargs=opt_args, calib_type=calib_type, calib_kwargs=calib_args, device=device)


def _run_model(model, loader, device, hooks_for, fn):
    """One pass of the float model over the calibration set with a forward hook on every linear in `hooks_for`;
    the hook hands (layer name, module, input) to fn."""
    hooks = []
    for name, module in model.named_modules():
        if isinstance(module, nn.Linear) and name in hooks_for:
            hooks.append(module.register_forward_hook(lambda mod, inp, out, n=name: fn(n, mod, inp[0])))
    model.eval()
    try:
        with torch.no_grad():
            for batch in loader:
                args = _move_to_device(batch[0], device)
                model(*args) if isinstance(args, tuple) else model(**args)
    finally:
        for h in hooks:
            h.remove()


def _trace_linears(model, linears, loader, src_dev, dst_dev):
    _run_model(model, loader, src_dev, linears, lambda n, mod, x: linears[n].trace(_move_to_device(x, dst_dev)))


def _smooth_linears(linears):
    for lin in linears.values():
        lin.smooth()


def _calib_linears(model, linears, loader, src_dev, dst_dev):
    _run_model(model, loader, src_dev, linears, lambda n, mod, x: linears[n].calibrate(_move_to_device(x, dst_dev)))
    for lin in linears.values():
        lin.finish_calibrate()


def _search_linears(model, linears, loader, src_dev, dst_dev, dump_search=False):
    """One candidate of the alpha search: per-chunk mean squared error of the quantised layer against the float
    layer's per-segment products, summed over the calibration set, handed to the optimizer's search_step."""
    err, float_linears = {k: None for k in linears}, {}

    def measure(n, mod, x):
        float_linears[n] = mod
        x = _move_to_device(x, dst_dev)
        real = linears[n].segment_forward(x, weight=_move_to_device(mod.weight.data, dst_dev))
        cur = linears[n].forward(x, chunked=True)
        d = [((r - c) ** 2).mean().item() for r, c in zip(real, cur)]
        err[n] = d if err[n] is None else [a + b for a, b in zip(err[n], d)]

    _run_model(model, loader, src_dev, linears, measure)
    for n in list(linears):
        w0 = _move_to_device(float_linears[n].weight.data, dst_dev)
        if linears[n].optimizer.search_step(err[n], origin_weight=w0):
            del linears[n]
    if dump_search:
        state = {k: {a: getattr(v.optimizer, a) for a in ("candidate_alphas", "alpha", "opt_err", "opt_alpha")}
                 for k, v in linears.items()}
        path = f"search_dump_{uuid.uuid4()}.pt"
        torch.save(state, path)
        print(f"[Search Linears] Dumped search results to {path}")


def _replace_linears(model, new_linears, device):
    for name, new in new_linears.items():
        parent = model
        *path, leaf = name.split(".")
        for part in path:
            parent = parent[int(part)] if isinstance(parent, (nn.ModuleList, nn.Sequential)) and part.isdigit() else getattr(parent, part)
        new = new.to(device)
        if isinstance(parent, (nn.ModuleList, nn.Sequential)) and leaf.isdigit():
            parent[int(leaf)] = new
        else:
            setattr(parent, leaf, new)


def quantize(model, calib_data_loader, config=None, tmp_device=None, verbose=False, example=None, dump_search=False,
             search_recovery_file=None, seg_map=None, dual_scale=None):
    """Returns `model` with its enabled nn.Linear layers replaced by calibrated SegmentLinear layers.

    calib_data_loader yields batches whose first element is the model's positional-argument tuple (or keyword dict).
    config: {"default": {...}, "<fnmatch pattern>": {...}} as in segquant/config.py:77-97; tmp_device: where the new
    layers are built and calibrated (they end up on the model's own device); example is accepted for signature
    compatibility and unused (it only feeds the pattern detector)."""
    src_dev = next(model.parameters()).device
    dst_dev = src_dev if tmp_device is None else tmp_device
    final_config = dict(config or default_quantize_config)
    final_config.setdefault("default", default_quantize_config["default"])
    if all(not final_config[k]["enable"] for k in final_config):
        return model
    linears = _get_all_linears(model, final_config["default"]["enable"], final_config)
    if verbose:
        print(f"get valid linear num [{len(linears)}]")
    dual = set(dual_scale or ())
    wants_seg = any(cfg.get("seglinear") for cfg in final_config.values())
    if wants_seg and seg_map is None:
        raise NotImplementedError("this build has no graph pattern detector: pass seg_map={layer name: {'seg_mode', 'chunks' | "
                                  "'chunksizes'}} (and dual_scale=[names]), or set seglinear: false")
    new = {}
    for name, seg_cfg in (seg_map or {}).items():
        if name not in linears:
            continue
        if not _layer_config(name, final_config).get("seglinear", True):
            if verbose:
                print(f"[INFO] Detect but disabled [{name}]")
            continue
        new[name] = _create_linear(linears.pop(name), name, seg_cfg, final_config, name in dual, dst_dev)
    for name, lin in linears.items():
        new[name] = _create_linear(lin, name, {"chunks": 1, "seg_mode": "weight"}, final_config, name in dual, dst_dev)

    to_smooth = {k: v for k, v in new.items() if v.opt_type in ("smooth", "svd")}
    to_search = {k: v for k, v in new.items() if getattr(v.optimizer, "search_alpha", False)}
    if search_recovery_file is not None:
        for k, st in torch.load(search_recovery_file, weights_only=False).items():
            if k in to_search:
                for a, val in st.items():
                    setattr(to_search[k].optimizer, a, val)
    if to_smooth:
        _trace_linears(model, to_smooth, calib_data_loader, src_dev, dst_dev)
    while to_search:
        _smooth_linears(to_search)
        _calib_linears(model, to_search, calib_data_loader, src_dev, dst_dev)
        _search_linears(model, to_search, calib_data_loader, src_dev, dst_dev, dump_search=dump_search)
    if to_smooth:
        _smooth_linears(to_smooth)
    _calib_linears(model, new, calib_data_loader, src_dev, dst_dev)
    _replace_linears(model, new, src_dev)
    if verbose:
        print(model)
    return model
