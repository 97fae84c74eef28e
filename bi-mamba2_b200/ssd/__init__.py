"""B200-native drop-in for the `ssd` package of Hprairie/Bi-Mamba2: the bidirectional SSD chunk scan operator
(`ssd.bi.ssd_combined.bimamba_chunk_scan_combined`) and the `ssd.modules.BiMamba2` layer built on it."""
from ssd.modules import BiMamba2, Mamba2
from ssd.version import __version__

__all__ = ["BiMamba2", "Mamba2", "__version__"]
