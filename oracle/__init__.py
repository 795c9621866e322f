"""CPU oracle for the tensor-parallel transformer layer forward.  TEST INFRASTRUCTURE ONLY.

Nothing under this package is part of the product: only the test-suite, the smoke check and
the CPU-baseline leg of the benchmark may import it, and only as the checker.  The product
(`energonai_b200`) never imports it and fails loudly when its CUDA library is missing.

Contents
--------
kernels_np.py   index-for-index NumPy restatements of the reference's CUDA kernels
                (energonai/kernel/cuda_native/csrc/*.cu).
layers.py       torch (fp32, CPU) restatement of the reference layer forward
                (energonai/model/{attention,mlp,endecoder,embedding,downstream,model_factory}.py)
                with an optional simulated tensor-parallel split.
inputs.py       seeded synthetic inputs / weights for the benchmark configurations.
ref_loader.py   imports the reference's own Python (only where the reference checkout and
                the colossalai stand-in are available) to pin the restatements.
colossalai_standin/  minimal stand-in for the third-party `colossalai` symbols the
                reference imports (tensor-parallel size 1).

Parity pin: layers.py is checked against the reference's own `energonai.model` code run on
CPU (tests/test_oracle_vs_reference.py, and the fixtures under tests/golden/ produced by
tests/golden/make_golden.py).  The CUDA-kernel restatements are checked against the known
answers derived from the reference's kernel-test fixtures (sequence lengths
[24,127,31,65,24,127,31,65], batch 8, padded length 128: tests/test_kernel/test_ft_transpose_pad.py:6-11)
and the identities its tests assert (tests/test_kernel/test_transpose_pad_fusion_kernel.py:63-79).
scale_mask_softmax and LayerNorm have no reference test: for those two the restatement is the pin.
"""
