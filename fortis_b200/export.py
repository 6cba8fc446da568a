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
