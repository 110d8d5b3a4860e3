"""B200-native (sm_100a) W8A8 linear layers for the Hunyuan3D-2.1 texture UNet.

The directory name contains a hyphen, so import the package with
``importlib.import_module("hunyuan3d-tools_b200")`` (the repository root on ``sys.path``);
sub-modules then import normally, e.g. ``pkg.quantize_utils`` and ``pkg.csrc.build``.
"""
