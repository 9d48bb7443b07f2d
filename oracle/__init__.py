"""CPU oracle: a restatement of the reference's torch golden functions.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package imports this module.
It is used by ``tests/``, by ``__graft_entry__.smoke()`` and by the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py`` as the checker and
the timed CPU arm; it is never the thing shipped.

The reference (hw-native-sys/pypto) defines numerics for its model examples by
plain-torch ``golden()`` functions.  Every function here cites the reference
file:line it restates.  Parts of the workload that the reference does not
contain (GQA with several KV heads, q_len > 1 with a causal draft mask, sigmoid
gate + top-k, FP8 with 128x128 block scales, shared expert) are marked
"parity unpinned": this oracle is then the only definition.

Pinning: ``tests/test_oracle_vs_reference.py`` AST-extracts the reference's own
``golden()`` bodies (they use torch/struct only) when the reference tree is
present and compares bit-for-bit; ``tests/golden/`` holds vectors produced by
those extracted functions so the pin travels to machines without the tree.
"""

from . import ep, ffn, gather, inputs, layer, moe, paged_attention  # noqa: F401
