// Forwarding header: the declarations live in topoanns/api.hpp.
#pragma once
#include "topoanns/api.hpp"
