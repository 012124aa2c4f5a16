"""CPU restatement of the reference's arithmetic for the QLoRA hot path. TEST INFRASTRUCTURE ONLY.

Nothing in the product (`claudemaxing_b200/`) imports this package. It exists so that the CUDA
kernels can be checked against the reference's own algorithm on the same seeded inputs:
`tests/`, `__graft_entry__.smoke()` and the `cpu_baseline` / `--impl reference` legs of
`bench.py` are its only users.

The reference is Python (torch + Triton) and has no CPU implementation of its own kernels; on CPU
its patches fall back to the installed HF/torch code. Each function here therefore restates either
the plain-torch reference function of the reference's own test for that op, or the kernel's
arithmetic step by step, and cites the file:line it follows.

How it is pinned: the reference's Triton kernels were executed with Triton's CPU interpreter in
the authoring container on seeded inputs and their outputs stored under `tests/golden/`
(`tests/golden/make_golden.py`); `tests/test_oracle_golden.py` checks every function here against
those vectors (bit-exact for NF4 and the dropout bits, within the reference's own tolerances for
the floating-point ops). The one part that stays unpinned is bitsandbytes' literal NF4 / dynamic
8-bit code tables and its quantiser, which are not in the reference tree nor in this environment:
`oracle.nf4.nf4_code_table` / `dynamic_map` / `quantize_nf4` are stand-ins built from the
published definition, and the dequantiser takes the tables as inputs, so dequant parity holds for
any tables.
"""
