"""From a torch module to the model blob the runtime loads: the role of the reference's export scripts plus weight
outlining (frontend/export_mlp.py:3-14, frontend/export_conv.py, driver/fortis_outline.py:13-35), without a compiler in
between: the layer list is read off the module, the weights off its state_dict.

    blob = fortis_b200.export.blob_from_torch(torch.nn.Sequential(...))
    open("model.fortis", "wb").write(blob)            # then FORTIS_MODEL=model.fortis, or fortis_load_model(path)

Supported: nn.Sequential (nested) of Linear / Conv3d (cubic kernel, stride 1, "same" padding) with ReLU / LeakyReLU /
Identity / Flatten-free activations between them, and residual blocks given as modules with attributes `body`
(a Sequential) whose output is added to the block's input (what the super-resolution nets of the reference use).
Anything else raises: a layer that would be silently dropped is worse than no export.
"""
import numpy as np

from .model import write_blob


def _np(t):
    return t.detach().cpu().numpy().astype(np.float32)


def layers_from_torch(module):
    """Layer dicts (W, b, act, slope, pad, save, add) in execution order."""
    import torch.nn as nn
    layers = []

    def set_act(kind, slope=0.0):
        if not layers:
            raise ValueError("an activation comes before the first layer")
        if layers[-1]["act"] != "none":
            raise ValueError("two activations in a row are not a layer sequence this runtime has a kernel for")
        layers[-1]["act"], layers[-1]["slope"] = kind, float(slope)

    def visit(m):
        if isinstance(m, nn.Sequential):
            for c in m:
                visit(c)
        elif isinstance(m, nn.Linear):
            b = _np(m.bias) if m.bias is not None else np.zeros(m.out_features, np.float32)
            layers.append(dict(W=_np(m.weight), b=b, act="none", slope=0.0))
        elif isinstance(m, nn.Conv3d):
            k = m.kernel_size
            if not (k[0] == k[1] == k[2]) or m.stride != (1, 1, 1) or m.dilation != (1, 1, 1) or m.groups != 1:
                raise ValueError("Conv3d must have a cubic kernel, stride 1, no dilation, one group")
            if m.padding != (k[0] // 2,) * 3:
                raise ValueError("Conv3d must keep the spatial extent (padding = kernel // 2)")
            b = _np(m.bias) if m.bias is not None else np.zeros(m.out_channels, np.float32)
            layers.append(dict(W=_np(m.weight), b=b, act="none", slope=0.0, pad=k[0] // 2))
        elif isinstance(m, nn.ReLU):
            set_act("relu")
        elif isinstance(m, nn.LeakyReLU):
            set_act("leaky", m.negative_slope)
        elif isinstance(m, nn.Identity):
            pass
        elif hasattr(m, "body") and isinstance(m.body, nn.Sequential):
            # residual block: out = in + body(in).  The layer in front remembers its output as the skip; the block's
            # last layer adds it (before its own activation, of which a residual body has none) and is the next skip.
            if not layers:
                raise ValueError("a residual block needs a layer in front of it")
            layers[-1]["save"] = True
            n0 = len(layers)
            visit(m.body)
            if len(layers) == n0 or layers[-1]["act"] != "none":
                raise ValueError("a residual body must end in a layer without activation")
            layers[-1]["add"] = True
            layers[-1]["save"] = True
        else:
            raise ValueError("no kernel for module %s" % type(m).__name__)

    visit(module)
    if not layers:
        raise ValueError("the module has no Linear or Conv3d layer")
    return layers


def blob_from_torch(module, in_div=None, out_mul=None, relu_mask=None) -> bytes:
    return write_blob(layers_from_torch(module), in_div=in_div, out_mul=out_mul, relu_mask=relu_mask)


def blob_from_state_dict(state_dict, acts, slope=0.0, prefix="") -> bytes:
    """A plain MLP from a state_dict with keys `<prefix><i>.weight` / `<prefix><i>.bias` (what nn.Sequential of Linear
    and activation modules saves); `acts` names the activation after each Linear ('none' | 'relu' | 'leaky')."""
    idx = sorted({int(k[len(prefix):].split(".")[0]) for k in state_dict if k.startswith(prefix) and k.endswith(".weight")})
    if len(idx) != len(acts):
        raise ValueError("%d Linear layers in the state_dict, %d activations given" % (len(idx), len(acts)))
    layers = []
    for i, act in zip(idx, acts):
        W = _np(state_dict["%s%d.weight" % (prefix, i)])
        b = state_dict.get("%s%d.bias" % (prefix, i))
        layers.append(dict(W=W, b=_np(b) if b is not None else np.zeros(W.shape[0], np.float32), act=act, slope=slope))
    return write_blob(layers)


# -----------------------------------------------------------------------------------------------------------------
# 2-D operator networks (NCHW): Conv2d, ConvTranspose2d, BatchNorm2d (inference), zero padding, MaxPool2d, nearest
# Upsample, activations, and channel concatenation of parallel convolutions on one input.  Everything that is algebra
# on the weights is folded here (what the reference's compiler does as graph rewrites, compiler/FortisFuse.cpp:309-356
# for the padding): BatchNorm into the preceding convolution, explicit padding into the following one, a transposed
# convolution into the convolution of the dilated input with the flipped kernel, a concatenation of convolutions of
# the same input into one convolution with stacked output channels.
# -----------------------------------------------------------------------------------------------------------------
def layers2d_from_torch(module, in_channels=None):
    """Layer dicts for fortis_b200.model.write_blob (op = 'conv2d' | 'maxpool2d' | 'upsample2d') in execution order.
    The module is traced with torch.fx, so its forward may be any straight-line composition of the supported modules
    and torch.cat(dim=1) of parallel convolutions."""
    import torch
    import torch.fx
    import torch.nn as nn
    gm = torch.fx.symbolic_trace(module)
    mods = dict(gm.named_modules())
    rec = {}                                   # fx node -> dict(parent, layer | None, pad)

    def conv_layer(W, b, stride, pad, dil=1, extra=(0, 0)):
        return dict(op="conv2d", W=W, b=b, stride=tuple(int(v) for v in stride), pad=tuple(int(v) for v in pad), dil=int(dil),
                    extra=tuple(int(v) for v in extra), act="none", slope=0.0)

    def pending_pad(node):
        """Explicit zero padding accumulated directly in front of `node`'s consumer; returns (source node, (ph, pw))."""
        ph = pw = 0
        while rec[node]["layer"] is None and rec[node].get("pad") is not None:
            l, r, t, b = rec[node]["pad"]
            if l != r or t != b:
                raise ValueError("only symmetric zero padding folds into a convolution")
            ph, pw = ph + t, pw + l
            node = rec[node]["parent"]
        return node, (ph, pw)

    def single_use(node):
        return len(node.users) == 1

    out_node = None
    for node in gm.graph.nodes:
        if node.op == "placeholder":
            rec[node] = dict(parent=None, layer=None)
        elif node.op == "output":
            out_node = node.args[0]
        elif node.op == "call_module":
            m, src = mods[node.target], node.args[0]
            if isinstance(m, nn.Conv2d):
                if m.dilation != (1, 1) or m.groups != 1 or isinstance(m.padding, str) or m.padding_mode != "zeros":
                    raise ValueError("Conv2d: dilation, groups and non-zero padding modes have no kernel here")
                src, (ph, pw) = pending_pad(src)
                b = _np(m.bias) if m.bias is not None else np.zeros(m.out_channels, np.float32)
                rec[node] = dict(parent=src, layer=conv_layer(_np(m.weight), b, m.stride, (m.padding[0] + ph, m.padding[1] + pw)))
            elif isinstance(m, nn.ConvTranspose2d):
                kh, kw = m.kernel_size
                if m.dilation != (1, 1) or m.groups != 1 or m.stride[0] != m.stride[1]:
                    raise ValueError("ConvTranspose2d: dilation, groups and anisotropic strides have no kernel here")
                if m.padding[0] > kh - 1 or m.padding[1] > kw - 1:
                    raise ValueError("ConvTranspose2d: padding larger than kernel - 1")
                if rec[src]["layer"] is None and rec[src].get("pad") is not None:
                    raise ValueError("zero padding in front of a transposed convolution does not fold")
                W = np.ascontiguousarray(_np(m.weight).transpose(1, 0, 2, 3)[:, :, ::-1, ::-1])     # (Cin,Cout,kh,kw) -> flipped (Cout,Cin,kh,kw)
                b = _np(m.bias) if m.bias is not None else np.zeros(m.out_channels, np.float32)
                rec[node] = dict(parent=src, layer=conv_layer(W, b, (1, 1), (kh - 1 - m.padding[0], kw - 1 - m.padding[1]), dil=m.stride[0],
                                                              extra=m.output_padding))
            elif isinstance(m, nn.BatchNorm2d):
                L = rec[src]["layer"]
                if L is None or L["op"] != "conv2d" or L["act"] != "none" or not single_use(src) or m.training:
                    raise ValueError("BatchNorm2d folds only into a convolution directly in front of it (eval mode)")
                g = _np(m.weight) if m.affine else np.ones(m.num_features, np.float32)
                beta = _np(m.bias) if m.affine else np.zeros(m.num_features, np.float32)
                k = (g.astype(np.float64) / np.sqrt(_np(m.running_var).astype(np.float64) + m.eps))
                W = (L["W"].astype(np.float64) * k[:, None, None, None]).astype(np.float32)
                b = ((L["b"].astype(np.float64) - _np(m.running_mean)) * k + beta).astype(np.float32)
                rec[node] = dict(parent=rec[src]["parent"], layer=dict(L, W=W, b=b))
            elif isinstance(m, (nn.ReLU, nn.LeakyReLU)):
                L = rec[src]["layer"]
                if L is None or L["op"] != "conv2d" or L["act"] != "none" or not single_use(src):
                    raise ValueError("an activation fuses only into a convolution directly in front of it")
                act = dict(act="relu", slope=0.0) if isinstance(m, nn.ReLU) else dict(act="leaky", slope=float(m.negative_slope))
                rec[node] = dict(parent=rec[src]["parent"], layer=dict(L, **act))
            elif isinstance(m, (nn.ZeroPad2d, nn.ConstantPad2d)):
                if isinstance(m, nn.ConstantPad2d) and float(m.value) != 0.0:
                    raise ValueError("only zero padding folds into a convolution")
                rec[node] = dict(parent=src, layer=None, pad=tuple(int(v) for v in m.padding))
            elif isinstance(m, nn.MaxPool2d):
                k, st = m.kernel_size, m.stride if m.stride is not None else m.kernel_size
                pad = m.padding if isinstance(m.padding, tuple) else (m.padding, m.padding)
                dil = m.dilation if isinstance(m.dilation, tuple) else (m.dilation, m.dilation)
                if pad != (0, 0) or dil != (1, 1) or m.ceil_mode:
                    raise ValueError("MaxPool2d: padding, dilation and ceil_mode have no kernel here")
                rec[node] = dict(parent=src, layer=dict(op="maxpool2d", k=k, stride=st))
            elif isinstance(m, nn.Upsample):
                sf = m.scale_factor
                sf = (sf, sf) if not isinstance(sf, (tuple, list)) else tuple(sf)
                if m.mode != "nearest" or sf is None or any(float(v) != int(v) for v in sf):
                    raise ValueError("Upsample: only nearest with an integer scale")
                rec[node] = dict(parent=src, layer=dict(op="upsample2d", scale=(int(sf[0]), int(sf[1]))))
            elif isinstance(m, nn.Identity):
                rec[node] = dict(parent=src, layer=None)
            else:
                raise ValueError("no kernel for module %s" % type(m).__name__)
        elif node.op == "call_function" and node.target is torch.cat:
            parts = list(node.args[0])
            dim = node.kwargs.get("dim", node.args[1] if len(node.args) > 1 else 0)
            Ls = [rec[p]["layer"] for p in parts]
            same = all(L is not None and L["op"] == "conv2d" and rec[p]["parent"] is rec[parts[0]]["parent"] and
                       L["W"].shape[1:] == Ls[0]["W"].shape[1:] and
                       all(L[k] == Ls[0][k] for k in ("stride", "pad", "dil", "extra", "act", "slope")) for p, L in zip(parts, Ls))
            if dim != 1 or not same:
                raise ValueError("torch.cat is supported along the channels of convolutions of one input with one geometry")
            rec[node] = dict(parent=rec[parts[0]]["parent"],
                             layer=dict(Ls[0], W=np.concatenate([L["W"] for L in Ls]), b=np.concatenate([L["b"] for L in Ls])))
        else:
            raise ValueError("no kernel for graph node %s %s" % (node.op, node.target))
    # linearise from the output back to the input
    layers, node = [], out_node
    while node is not None:
        r = rec[node]
        if r["layer"] is None and r.get("pad") is not None:
            raise ValueError("zero padding must be followed by a convolution")
        if r["layer"] is not None:
            layers.append(r["layer"])
        node = r["parent"]
    layers.reverse()
    if not layers:
        raise ValueError("the module has no supported layer")
    c = in_channels
    for L in layers:                                   # channel counts of the layers without weights
        if L["op"] == "conv2d":
            c = L["W"].shape[0]
        else:
            if c is None:
                raise ValueError("give in_channels: the network starts with a layer that has no weights")
            L["channels"] = c
    return layers


def blob2d_from_torch(module, in_channels=None) -> bytes:
    return write_blob(layers2d_from_torch(module, in_channels=in_channels))
