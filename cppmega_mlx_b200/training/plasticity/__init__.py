from .dash import dash_step, dash_step_model, dash_step_tree
from .fire import apply_fire, newton_schulz, reset_optimizer_states_for_fired, spectral_norm_power_iter
from .redo import ReDoDiagnostics, ffn_layer_map, recycle_dormant_neurons
