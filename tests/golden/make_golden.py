"""Generates tests/golden/*.npz from the COMPILED REFERENCE (oracle/_ref/libedge0_ref.so, built by
`make -C oracle ref` from the reference's own ggml CPU sources).  Run where the reference tree is present:

    python tests/golden/make_golden.py [case ...]      (no names: every case and the known-answer file)

Each fixture holds the seeded inputs that cannot be regenerated without the reference (Q3_K weight bytes)
plus every observable output of the layer, so the restatement and the CUDA path can be checked against the
reference's own results on machines that do not have the reference.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from edge0_b200 import workloads as W  # noqa: E402
from edge0_b200.capi import TYPE_NVFP4, TYPE_Q3_K  # noqa: E402
from oracle import oracle as O  # noqa: E402

CASES = {
    # name: (config, tokens, bf16 activations)
    "q3k_small": (W.small_config(TYPE_Q3_K, n_embd=256, n_expert=8, top_k=2, n_ff=256, seed=11), 4, False),
    "nvfp4_small": (W.small_config(TYPE_NVFP4, n_embd=256, n_expert=8, top_k=2, n_ff=256, seed=12), 4, True),
    "nvfp4_small_bias": (W.small_config(TYPE_NVFP4, n_embd=512, n_expert=16, top_k=4, n_ff=256, router_bias=True, seed=13), 6, True),
    "nvfp4_small_latent": (W.small_config(TYPE_NVFP4, n_embd=512, n_latent=256, n_expert=16, top_k=4, n_ff=256, seed=14), 5, True),
    "nvfp4_small_shexp": (W.small_config(TYPE_NVFP4, n_embd=512, n_expert=16, top_k=4, n_ff=256, n_ff_shexp=512, seed=15), 6, False),
}


# a GGUF file with one MoE block (and its shared expert), written by the reference's gguf writer: input of the reader's tests
GGUF_CASE = dict(config=W.small_config(TYPE_NVFP4, n_embd=64, n_expert=8, top_k=2, n_ff=64, n_ff_shexp=128, seed=16, tensor_scales=False), layer=5,
                 file="moe_block_nvfp4.gguf")


def write_gguf_fixture(ref, path=None):
    cfg = GGUF_CASE["config"]
    layer = W.make_layer(cfg)
    path = path or os.path.join(HERE, GGUF_CASE["file"])
    ref.write_moe_gguf(path, layer=GGUF_CASE["layer"], wtype=cfg.wtype, router_w=layer.router_w, gate=layer.gate, up=layer.up, down=layer.down,
                       top_k=cfg.top_k, sh_gate=layer.gate_shexp, sh_up=layer.up_shexp, sh_down=layer.down_shexp, sh_gate_inp=layer.gate_inp_shexp)
    return path


def main():
    ref = O.reference()
    print("reference ISA:", ref.isa())
    q3k = lambda w: ref.quantize(TYPE_Q3_K, w)
    only = sys.argv[1:]
    if not only or "gguf" in only:
        p = write_gguf_fixture(ref)
        print(os.path.basename(p), os.path.getsize(p) // 1024, "KiB")
    for name, (cfg, T, bf16) in CASES.items():
        if only and name not in only:
            continue
        layer = W.make_layer(cfg, quantize_q3k=q3k)
        x = W.make_tokens(cfg, T, bf16=bf16)
        r = ref.moe_layer(x=x, n_threads=2, **layer.checker_kwargs())
        out = dict(x=x, logits=r.logits, probs=r.probs, ids=r.ids, weights=r.weights, hidden=r.hidden, down_out=r.down_out,
                   moe_out=r.moe_out, out=r.out)
        if cfg.n_ff_shexp:
            out.update(shexp_gated=r.shexp_gated)
        if cfg.wtype == TYPE_Q3_K:   # cannot be regenerated without the reference quantiser
            out.update(gate=layer.gate, up=layer.up, down=layer.down)
        else:                        # regenerated from the seed; keep a checksum to detect drift
            out.update(weight_sum=np.array([int(layer.gate.astype(np.uint64).sum()), int(layer.up.astype(np.uint64).sum()),
                                            int(layer.down.astype(np.uint64).sum())], dtype=np.uint64))
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, **out)
        print(name, os.path.getsize(path) // 1024, "KiB", "out rms", float(np.sqrt(np.mean(r.out ** 2))))

    if only:
        return
    # known-answer vectors for the codecs and the dot products (reference functions called directly)
    rng = np.random.default_rng(5)
    kat = {}
    for wname, wt, K in (("q3k", TYPE_Q3_K, 512), ("nvfp4", TYPE_NVFP4, 512)):
        w = rng.normal(0, 0.02, (8, K)).astype(np.float32)
        if wt == TYPE_NVFP4:
            w[0] *= 2000.0
        x = rng.normal(0, 1, (3, K)).astype(np.float32)
        wq = ref.quantize(wt, w)
        aq = ref.quantize_activation(wt, x)
        dots = np.array([[ref.vec_dot(wt, K, wq[i], aq[j]) for j in range(3)] for i in range(8)], dtype=np.float32)
        kat.update({f"{wname}_w": w, f"{wname}_x": x, f"{wname}_wq": wq, f"{wname}_aq": aq, f"{wname}_dots": dots,
                    f"{wname}_deq": ref.dequantize(wt, wq, K)})
    np.savez_compressed(os.path.join(HERE, "kat.npz"), **kat)
    print("kat.npz written")


if __name__ == "__main__":
    main()
