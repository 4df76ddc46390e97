"""khan_b200: the ANI-1 featurizer path of khan on B200 -- CUDA kernels behind a C ABI, with the
reference's op names (``ani_mod``), dataset type (``RawDataset``) and trainer front end."""
from .data.dataset import RawDataset  # noqa: F401


def __getattr__(name):
    # the trainer pulls in torch; import it on demand
    if name in ("TrainerMultiTower", "TrainerMultiGPU"):
        from .training import trainer_multi_tower as t
        return getattr(t, name)
    if name == "FlatNadam":
        from .training.optim import FlatNadam
        return FlatNadam
    if name == "FusedTrainStep":
        from .training.fused_step import FusedTrainStep
        return FusedTrainStep
    if name == "EnergyForces":
        from .inference import EnergyForces
        return EnergyForces
    if name in ("BatchFeeder", "PackedDataset"):
        from .data import feeder
        return getattr(feeder, name)
    raise AttributeError(name)
