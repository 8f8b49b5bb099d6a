// Shim: intentionally empty.
#pragma once
