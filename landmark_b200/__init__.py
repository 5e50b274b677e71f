"""landmark_b200: the GridNeRF render path of InternLandMark/LandMark on B200 (sm_100a).

Importing the package does not load the CUDA library; ``landmark_b200.gridnerf`` (and what
builds on it) does, and raises if the library has not been built.
"""

__all__ = ["scenes", "build"]
