"""CPU oracle for the batch-1 speculative decode path -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.

A restatement, in plain torch-on-CPU / numpy / Python integers, of the algorithm the reference
project (manaspros/qengine) defines for this path:

  w4.py     int4 group-128 wire format: quantiser, packer, dequantiser  (python/qengine/quant.py)
  model.py  the hybrid Gated-DeltaNet / gated-attention model, one token per step, with every
            bf16 rounding point of the reference torch model               (python/qengine/reference.py)
  spec.py   the speculative cycle the reference only has as CUDA + engine code: accept, commit,
            mtp_select, the pass ordering and MTP positions   (csrc/basic.cu:241-307,
            python/qengine/engine.py:468-520, 558-637)

Only tests/, __graft_entry__.smoke() and the CPU-baseline / reference arm of bench.py may import
this package, and only as the checker or as the timed CPU baseline. Nothing under qengine_b200/
imports it; the product path fails loudly when its CUDA library is missing.

Parity pinning: the reference stores no golden vectors of its own for this path (all of its
checks compare against torch at test time on weights that are not available offline). The
oracle is therefore pinned against outputs of the reference's own Python modules
(`qengine.reference`, `qengine.quant`) run on CPU on seeded inputs; those outputs are committed
under tests/golden/ together with the script that produced them (tests/golden/make_golden.py),
and tests/test_oracle_golden.py checks every oracle function against them.
"""
