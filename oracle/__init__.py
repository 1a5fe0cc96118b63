"""CPU restatement of BitsMoE's quantized-expert forward path.  TEST INFRASTRUCTURE.

Nothing in the shipped package imports this directory.  It exists so that the
tests, the smoke check and the ``cpu_baseline`` leg of the benchmark have an
independent statement of what the reference computes:

  bitplane.py   int8 codes <-> uint32 bit-planes
                (bitsmoe/quant/bitpack/bitpack_cuda_kernel.cu:81-121, :157-196;
                 offsets bitsmoe/quant/bitpack/__init__.py:22)
  quantize.py   quantize_symmetric / dequantize_symmetric
                (bitsmoe/quant/quantizer.py:30-84, :116-128)
  packer.py     slab / tile / stage / micro payload layout and the ten buffers
                per matrix (bitsmoe/quant/packer.py:169-207, :210-374, :517-724),
                the decoder the kernels imply (mlp_forward.cu:203-275) and the
                layout self-check (packer.py:377-460)
  forward.py    router, routing build, packed forward in fp32 and in the
                reference tensor-core path's fp16 rounding, down basis
                (bitsmoe/models/qwen3moe/bitsmoe_block.py:39-98,
                 bitsmoe/models/base_block.py:258-289, :409-414,
                 bitsmoe/algorithms/cpp/mlp_forward.cu:691-790, :1478-1501,
                 :2036-2066)

Pinning.  The reference ships no golden vectors and no forward test; its only
known-answer check is ``validate_runtime_layout``.  This oracle is pinned by
  (1) fixtures under tests/golden/ produced by importing the reference's own
      Python (quantize_symmetric, the layout reorder, the slab packer and
      validate_runtime_layout run on this oracle's buffers) -- see
      tests/golden/make_golden.py;
  (2) the reference's CUDA extensions compiled unmodified for sm_100a into
      oracle/_ref/ (build_ref.py) and run in the GPU tests: bit-plane pack /
      unpack bit-exact, moe_packed_forward within the stated tolerance.
"""
