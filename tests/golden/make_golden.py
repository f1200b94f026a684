"""Records golden fixtures from the reference project's own CUDA kernels.

Run on a machine with a GPU after oracle/build_ref.sh has produced
oracle/_ref/libref_grad.so (the reference sources compiled unmodified):

    python tests/golden/make_golden.py [output_dir]

Each fixture is a small .npz holding the input and the reference kernels'
output for one entry point; tests/test_oracle.py checks the CPU oracle
against them without a GPU.  Inputs avoid subnormal values: the reference
library is built with --use_fast_math, which flushes them, while its CPU codec
(the parity authority) does not.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, ".."))
sys.path.insert(0, os.path.join(HERE, "..", ".."))

import oracle            # noqa: E402  (input generator only)
import reference_kernels as rk  # noqa: E402
import vectors           # noqa: E402


def main(out_dir: str) -> None:
    os.makedirs(out_dir, exist_ok=True)

    def save(name, **arrays):
        np.savez_compressed(os.path.join(out_dir, name + ".npz"), **arrays)
        print("wrote", name)

    seeded = oracle.generate_gradient(4096, 0xB2000000, 0, subnormals=0)
    for block in (0, 32, 96, 128):
        for tag, source in (("closed515", vectors.codec_vector(515)), ("seeded4096", seeded)):
            payload, scales, decoded = rk.codec(source, block)
            save(f"codec_{tag}_block{block}", kind="codec", block=block, source=source,
                 payload=payload, scales=scales, decoded=decoded)
    tail = vectors.tail_max_vector(300137)[-4099:].copy()
    payload, scales, decoded = rk.codec(tail, 0)
    save("codec_tailmax4099_block0", kind="codec", block=0, source=tail, payload=payload, scales=scales,
         decoded=decoded)

    poisoned = vectors.codec_vector(515)
    poisoned[130] = np.inf
    poisoned[400] = np.nan
    payload, scales = rk.pack_bfp8_block(poisoned)
    save("pack_bfp8_block_poisoned515", kind="pack_bfp8_block", source=poisoned, payload=payload, scales=scales)
    payload, scales = rk.pack_bfp8_block(seeded)
    save("pack_bfp8_block_seeded4096", kind="pack_bfp8_block", source=seeded, payload=payload, scales=scales)

    other = oracle.generate_gradient(4096, 0xB2000000, 1, subnormals=0)
    pa, sa = rk.pack_bfp8_block(seeded)
    pb, sb = rk.pack_bfp8_block(other)
    reduced, sq = rk.block_transport_sum(pa, sa, pb, sb)
    save("block_transport_sum_seeded4096", kind="block_transport_sum", payload0=pa, scales0=sa, payload1=pb,
         scales1=sb, reduced=reduced, squared_sum=sq)

    a_bits, b_bits = rk.pack_bf16(seeded), rk.pack_bf16(other)
    save("pack_bf16_seeded4096", kind="pack_bf16", source=seeded, packed=a_bits)
    reduced, sq = rk.bf16_transport_sum(a_bits, b_bits)
    save("bf16_transport_sum_seeded4096", kind="bf16_transport_sum", a=a_bits, b=b_bits, reduced=reduced,
         squared_sum=sq)

    for n in (1, 257, 515):
        source = vectors.reducer_vector(n, 0.0, 0.25, 2.75)
        g, payload, scale, flag, sq = rk.gradient_publish(source)
        save(f"gradient_publish_{n}", kind="gradient_publish", source=source, gradient_after=g, payload=payload,
             scale=scale, finite_status=flag, squared_sum=sq)


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "recorded"))
