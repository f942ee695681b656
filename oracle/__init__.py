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
  golden vector and no test that pins metadata values.  The restatement in
  sched_meta.py is pinned against outputs of the reference itself: the
  reference's own kernel
  (csrc/smxx/decode/get_decoding_sched_meta/get_decoding_sched_meta.cu,
  compiled unmodified into oracle/_ref/ by oracle/build_ref.py) runs beside it
  in tests/test_gpu_sched_reference.py on the hand-derived known answers and on
  about 270 random dense and sparse cases, value for value.  Where that library
  has not been built, the known answers (tests/golden/
  sched_meta_known_answers.json) and the schedule properties remain.
* split-KV combine: the reference's own kernel (csrc/smxx/decode/combine/
  combine.cu) is built into the same library and compared with this
  repository's kernel in the same test file.
"""
