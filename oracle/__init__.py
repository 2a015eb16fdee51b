"""CPU oracle for the LoRA fine-tuning step.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package imports this
directory; it is the checker used by `tests/`, by `__graft_entry__.smoke()`
and by the `cpu_baseline` / `--impl reference` legs of `bench.py`.

Two layers:

* `oracle.lora_step`  - whole-step restatement (forward, masked per-sequence
  mean cross-entropy, autograd backward, gradient mean over ranks, global
  norm, clipping, AdamW) in plain f32 PyTorch on the CPU.  It follows the
  reference's own CPU restatement of this path,
  `scripts/gen_gradient_fixtures.py:131-195`, parametrised over the model
  config, plus the update rule of
  `ferrotensor-backend/src/shaders/kernels.wgsl:355-387` and the host logic of
  `ferrotensor-trainer/src/lib.rs:296-360,426-534,676-752`.
* `oracle.kernels`    - per-kernel loops following the CPU helpers of
  `ferrotensor-backend/tests/gpu_kernels.rs:80-228,1300-1318,1513-1545`.

Parity pins (all checked by `tests/test_oracle_golden.py`):
  1. the four gradient-parity cases of the reference
     (`ferrotensor-graph/tests/fixtures/gradient_parity`): loss, logits and
     every gradient tensor, tolerance 1e-4 + 1e-3*|expected|;
  2. the bit-exact xorshift64* weight generator of
     `ferrotensor-graph/tests/common/mod.rs:66-161`;
  3. `lora_seed` known answers (`ferrotensor-graph/src/model_builder.rs:869-876`);
  4. the 40-step loss trajectory printed in
     `ferrotensor-trainer/examples/lora_finetune_tiny.rs:12-29`;
  5. LR-schedule values (`ferrotensor-autograd/src/lib.rs:1914-1939`).
"""
