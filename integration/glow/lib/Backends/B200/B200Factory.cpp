#include "B200Backend.h"

namespace glow {
REGISTER_GLOW_BACKEND_FACTORY(B200Factory, B200Backend);
} // namespace glow
