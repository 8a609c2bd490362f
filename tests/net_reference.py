"""CPU restatement of what apnn_tc_b200.nets computes, built only from oracle functions.

Test infrastructure.  Network-level outputs are project-defined (the reference's model
programs never check theirs): each layer is the pinned accumulator of the oracle followed by
the oracle's +-1 correction, 2x2 maximum, residual add and threshold requantisation.
"""
import numpy as np

import oracle


def forward_reference(spec, params, images, threads=8):
    """images: float32 [B, H, W, C].  Returns (logits [B, PAD128(classes)] -- float32 with float_logits, else
    int32 --, levels, values)."""
    a = spec.a_bit
    B = images.shape[0]
    first8 = spec.first_bits == 8
    lv0 = oracle.quantize(images, 8 if first8 else a)
    cp = params[spec.layers[0].name].shape["cinp"]   # stored channels of the image (zero-padded)
    x0 = np.zeros(images.shape[:3] + (cp,), dtype=np.uint32)
    x0[..., : spec.image_channels] = lv0
    levels = {None: x0}
    values = {}
    prev = None
    for ls in spec.layers:
        src = ls.src or prev
        p = params[ls.name]
        if ls.kind == "conv" and src is None and first8:
            # the image at 8 bits, re-centred, times the -1/+1 filter (oracle.centred_first_layer)
            v = oracle.centred_first_layer(p.weight_planes, levels[None], spec.image_channels, stride=ls.stride,
                                           threads=threads)
            if ls.pool == 2:
                v = oracle.pool2x2(v, 2)
        elif ls.kind == "conv":
            x = levels[src]
            pad = (ls.R - 1) // 2
            xp = np.zeros((B, x.shape[1] + 2 * pad, x.shape[2] + 2 * pad, x.shape[3]), dtype=np.uint32)
            xp[:, pad:pad + x.shape[1], pad:pad + x.shape[2]] = x
            X = oracle.pack_levels(xp, a)
            acc = oracle.conv_popc(p.weight_planes, X, stride=ls.stride, threads=threads)
            v = oracle.signed_correct(acc, oracle.conv_window_sums(X, ls.R, ls.stride), 0)
            if ls.pool == 2:
                v = oracle.pool2x2(v, 2)
        else:
            x = levels[src].reshape(B, -1)
            X = oracle.pack_levels(x, a)                       # activations are the first GEMM operand
            acc = oracle.gemm_popc(X, p.weight_planes, threads=threads)
            v = oracle.signed_correct(acc, oracle.row_sums(X), 0)
        if ls.residual_from:
            v = v + values[ls.residual_from]
        values[ls.name] = v
        if ls.quantise:
            levels[ls.name] = oracle.levels(v, a, 2, p.thresholds).astype(np.uint32)
        prev = ls.name
    last = spec.layers[-1].name
    logits = values[last]
    if params[last].affine is not None:
        logits = oracle.affine_f32(logits, params[last].affine[0], params[last].affine[1])
    return logits, levels, values
