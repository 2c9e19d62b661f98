"""mummu_b200 — the OLMoE top-k-routed SwiGLU expert bank of physics515/Mummu, written for B200
(sm_100a) behind a C ABI (include/mummu_cuda.h).  Importing `mummu_b200.moe` loads the CUDA
library; there is no CPU fallback."""
__all__ = ["moe", "q4k", "synth", "build"]
