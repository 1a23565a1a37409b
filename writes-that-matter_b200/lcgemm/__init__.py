"""lcgemm for B200: the rank-7 bilinear GEMM path of the LLM MLP prefill, hand-written for sm_100a.

Same layout as the reference package (``lcgemm/__init__.py:10-24``):

``scheme``        the decomposition and its epilogue plan (host, exact integers)
``planes``        operand-plane contract: offline B planes, A planes
``chain_gauge``   the interleaved-K gauge the chained epilogue emits in
``ops``           torch-tensor front end of the C ABI (``include/lcgemm_b200.h``)
``seams/``        ``GateUpPlan`` / ``DownPlan`` / ``build_chain``: what the model calls
``integrate/``    the vLLM swap: custom ops, the layer forward, arm/install
``layer``         one MLP layer in its arms: the rank-7 chain, the stock layer on the dense tcgen05
                  GEMM or on cuBLAS (the comparison arms), a layer call as one CUDA graph replay
``tp``            tensor-parallel MLP (column-parallel gate_up, row-parallel down, exchange over peer
                  memory or one all-reduce)
``streaming``     host-to-host streaming of batches through a layer (copies overlapped with compute)
``model``         a random-init dense decoder for end-to-end prefill comparisons

The device code is ``csrc/*.cu`` behind one shared library; nothing here falls
back to another implementation when that library is missing.
"""

__version__ = "0.1.0"
