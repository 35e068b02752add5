#pragma once
#include <nlohmann/json.hpp>
