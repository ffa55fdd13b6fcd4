"""CPU oracle of the quantized basecaller layer path. TEST INFRASTRUCTURE ONLY: imported by
tests/, by __graft_entry__.smoke() and by the cpu_baseline / reference legs of bench.py; the
product (src/, fluke_b200/) never imports it.

`oracle.port`  numpy front end of oracle/liboracle.so (the C restatement fluke_oracle.c)
`oracle.ref`   loaders for oracle/_ref/*.so (the reference's own sources compiled unmodified)
"""
