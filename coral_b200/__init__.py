"""coral_b200: B200-native (sm_100a) batched graph beam search behind CORAL's search API.

`coral_b200.capi` binds the C ABI (include/coral_b200.h); `coral_b200.synth` makes
seeded synthetic inputs.  Importing the package does not build or load anything.
"""
__all__ = ["capi", "synth", "build"]
