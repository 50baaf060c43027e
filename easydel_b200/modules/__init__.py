"""Model families. Importing this package registers every family with the registry."""

from . import llama  # noqa: F401
from .llama import *  # noqa: F401,F403
from . import families  # noqa: F401
from .families import *  # noqa: F401,F403
from . import families_classic  # noqa: F401
from .families_classic import *  # noqa: F401,F403
from . import mamba  # noqa: F401
from .mamba import *  # noqa: F401,F403
from . import families_extra  # noqa: F401
from .families_extra import *  # noqa: F401,F403
from .auto import *  # noqa: F401,F403
from . import roberta  # noqa: F401
from .roberta import *  # noqa: F401,F403
from . import vision, llava  # noqa: F401
from .vision import *  # noqa: F401,F403
from .llava import *  # noqa: F401,F403
from . import whisper  # noqa: F401
from .whisper import *  # noqa: F401,F403
from . import gemma3, aya_vision  # noqa: F401
from .gemma3 import *  # noqa: F401,F403
from .aya_vision import *  # noqa: F401,F403
from . import pixtral, mistral3  # noqa: F401
from .pixtral import *  # noqa: F401,F403
from .mistral3 import *  # noqa: F401,F403
from . import qwen2_vl  # noqa: F401
from .qwen2_vl import *  # noqa: F401,F403
from . import qwen3_vl  # noqa: F401
from .qwen3_vl import *  # noqa: F401,F403
from . import rwkv  # noqa: F401
from .rwkv import *  # noqa: F401,F403
from . import glm4v  # noqa: F401
from .glm4v import *  # noqa: F401,F403
from . import gemma4  # noqa: F401
from .gemma4 import *  # noqa: F401,F403
from . import qwen3_omni_moe  # noqa: F401
from .qwen3_omni_moe import *  # noqa: F401,F403
from . import kimi_vl  # noqa: F401
from .kimi_vl import *  # noqa: F401,F403
from . import llama4  # noqa: F401
from .llama4 import *  # noqa: F401,F403

# The halves of composite checkpoints under the model types their own configs carry.
from ..infra.factory import registry as _registry  # noqa: E402

for _alias, _target in {
    "qwen2_vl_text": "qwen2", "qwen3_vl_text": "qwen3", "qwen3_vl_moe_text": "qwen3_moe",
    "qwen3_vl_moe_vision": "qwen3_vl_vision", "glm4v_moe_text": "glm4_moe", "glm4v_moe_vision": "glm4v_vision",
    "qwen3_omni_moe_text": "qwen3_moe", "qwen3_omni_moe_vision_encoder": "qwen3_vl_vision",
}.items():
    _registry.alias(_alias, _target)

from . import aliases  # noqa: E402,F401
from .aliases import *  # noqa: E402,F401,F403
