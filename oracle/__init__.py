"""CPU restatement of the reference's MLA decode / sparse-prefill algorithms.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package may import this
directory: it is the checker for the CUDA path (tests, the smoke check and the
CPU-baseline leg of the benchmark), never the thing that is measured or
shipped.

Every function cites the reference file:line it restates (paths are relative
to the deepseek-ai/FlashMLA project root).

Pinning status
--------------
* attention / quantisation oracles: pinned against outputs of the reference's
  own torch code (tests/ref.py, tests/quant.py,
  tests/test_flash_mla_dense_decoding.py::reference_torch) that were generated
  by importing those files unchanged; the vectors and the generating script
  live in tests/golden/.
* tile-scheduler metadata: the reference holds no CPU implementation, no
  golden vector and no test that pins metadata values, so the restatement in
  sched_meta.py follows the CUDA source line by line and is pinned only by two
  hand-derived known answers and by structural invariants -- "parity unpinned"
  by the reference's own tests.
"""
