// The json copy bundled with cudnn-frontend ships json.hpp only; the reference includes the forward-declaration
// header of the same library in one place. The full header declares everything the forward header does.
#pragma once
#include <nlohmann/json.hpp>
