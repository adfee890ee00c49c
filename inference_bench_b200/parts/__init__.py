"""Parts of a decoder. Importing the package registers the standard parts."""
from . import base, plan, standard, latent, experts, recurrent, canon, shift, scan, parallel, loop, sigmoid  # noqa: F401
