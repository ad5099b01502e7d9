// Part of the GLM stand-in (test infrastructure): every name lives in glm/glm.hpp.
#pragma once
#include "../glm.hpp"
