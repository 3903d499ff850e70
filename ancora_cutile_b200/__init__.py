"""B200-native (sm_100a) Muon + AdamW hybrid optimizer step with the Python API of
ancora-cutile's ``ancora/optim`` package.  The arithmetic runs in libancora_b200.so
(hand-written CUDA behind a C ABI, include/ancora_b200.h) called through ctypes; there
is no PyTorch, no Triton and no CPU fallback in this package."""
from ._lib import AncoraError, LIB_PATH
from .buffers import Context, DBuf, Event, PinnedArray, dev_ptr, get_context, set_device
from .adamw import AdamW, ResidentAdamW
from .muon import (BatchedProjMuon, DeviceMuon, ExpertMuonScratch, Muon, MuonPlan, MuonScratch,
                   ResidentMuon)
from .muon_ns import (PE_SCHEDULE, newton_schulz_resident, newton_schulz_resident_e,
                      set_polar_express)
from .hybrid import HybridOptimizer, default_is_muon
from .resident import ResidentHybrid

__all__ = ["AncoraError", "LIB_PATH", "Context", "DBuf", "Event", "PinnedArray", "dev_ptr",
           "get_context", "set_device", "AdamW", "ResidentAdamW", "BatchedProjMuon", "DeviceMuon",
           "ExpertMuonScratch", "Muon",
           "MuonPlan", "MuonScratch", "ResidentMuon", "PE_SCHEDULE", "newton_schulz_resident",
           "newton_schulz_resident_e", "set_polar_express", "HybridOptimizer", "default_is_muon",
           "ResidentHybrid"]
