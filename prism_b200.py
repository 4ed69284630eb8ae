"""Import name of the package that lives in the directory `startlux-prism_b200/` (a hyphen cannot be imported):
`import prism_b200` and `from prism_b200 import w8a8, quant, w4a8, mxfp4, tp` resolve to the modules in that directory."""
import os as _os

__path__ = [_os.path.join(_os.path.dirname(_os.path.abspath(__file__)), "startlux-prism_b200")]
with open(_os.path.join(__path__[0], "__init__.py")) as _f:
    exec(compile(_f.read(), _os.path.join(__path__[0], "__init__.py"), "exec"))
del _f
